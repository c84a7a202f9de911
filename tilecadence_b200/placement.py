"""Solve shared-memory handoff offsets for the B200 attention kernels.

Same declarative surface as ``tilecadence/placement.py`` (``Region`` :13-19, ``Handoff`` :22-28,
``HANDOFFS`` :31-44, ``replay`` :47-62, ``solve`` :65-103, CLI :106-115): a donor byte range that a
kernel releases at a known step of a short timeline, and recipient regions (size, alignment,
half-open live interval) that must be packed into it without overlapping in time x address. The
result dictionary has the reference's schema and the reference's objective: minimum recipient
address high-water, then minimum offset of the first region.

What changed for sm_100a is the donor geometry (the kernels' shared-memory maps) and the solver:
the reference states the problem to OR-tools CP-SAT; here the optimum is found by exact
enumeration. Any packing can be slid down to a "first-fit" packing without raising either
objective term, and every first-fit packing is produced by placing the regions in some order at
the lowest aligned conflict-free address, so trying every order is exhaustive.
"""
from __future__ import annotations

import argparse
from dataclasses import asdict, dataclass
from itertools import permutations
import json
from pathlib import Path


@dataclass(frozen=True)
class Region:
    name: str
    size_bytes: int
    alignment_bytes: int
    start: int
    end: int


@dataclass(frozen=True)
class Handoff:
    donor_name: str
    donor_offset_bytes: int
    donor_bytes: int
    donor_release: int
    regions: tuple[Region, ...]
    timeline: tuple[str, ...]


# Donors on B200:
#   prefill  K stage 0 of the 2-stage K ring (32 KiB at byte 65536 of the CTA arena, after the two
#            32 KiB Q tiles); the ring index is chosen so the last QK^T always reads stage 0.
#   decode   the V half (16 KiB at byte 0) of stage 0 of the K/V ring; the last tile always uses it.
# Recipients keep the reference's sizes, alignments and live intervals.
HANDOFFS = {
    "prefill": Handoff(
        "terminal_K", 64 * 1024, 32 * 1024, 1,
        (Region("head0_lse", 512, 128, 1, 3),
         Region("head1_lse", 512, 128, 1, 3)),
        ("last_K_read", "K_readers_released_and_epilogue_scatter", "CTA_publish_and_export"),
    ),
    "decode": Handoff(
        "terminal_V", 0, 16 * 1024, 1,
        (Region("output_tile", 2048, 16, 1, 3),
         Region("row_lse", 16, 16, 1, 3)),
        ("last_V_read", "V_readers_released_and_epilogue_scatter", "CTA_publish_and_export"),
    ),
}


def replay(handoff: Handoff, offsets: dict[str, int]) -> None:
    """Independently check half-open times and byte ranges."""
    donor_lo = handoff.donor_offset_bytes
    donor_hi = donor_lo + handoff.donor_bytes
    steps = len(handoff.timeline)
    placed = []
    for region in handoff.regions:
        lo = offsets[region.name]
        hi = lo + region.size_bytes
        time_ok = handoff.donor_release <= region.start < region.end <= steps
        bytes_ok = donor_lo <= lo < hi <= donor_hi and lo % region.alignment_bytes == 0
        if not (time_ok and bytes_ok):
            raise ValueError(f"Invalid time/address placement for {region.name}")
        for other, other_lo in placed:
            live_together = max(region.start, other.start) < min(region.end, other.end)
            if live_together and max(lo, other_lo) < min(hi, other_lo + other.size_bytes):
                raise ValueError(f"Live byte ranges overlap for {region.name} and {other.name}")
        placed.append((region, lo))


def _align_up(value: int, step: int) -> int:
    return -(-value // step) * step


def _first_fit(handoff: Handoff, order) -> dict[str, int] | None:
    donor_lo = handoff.donor_offset_bytes
    donor_hi = donor_lo + handoff.donor_bytes
    placed: list[tuple[Region, int]] = []
    for region in order:
        offset = _align_up(donor_lo, region.alignment_bytes)
        moved = True
        while moved:
            moved = False
            for other, other_lo in placed:
                if max(region.start, other.start) >= min(region.end, other.end):
                    continue
                other_hi = other_lo + other.size_bytes
                if max(offset, other_lo) < min(offset + region.size_bytes, other_hi):
                    offset = _align_up(other_hi, region.alignment_bytes)
                    moved = True
        if offset + region.size_bytes > donor_hi:
            return None
        placed.append((region, offset))
    return {region.name: offset for region, offset in placed}


def solve(handoff: Handoff) -> dict:
    for region in handoff.regions:
        if region.size_bytes <= 0 or region.alignment_bytes <= 0:
            raise ValueError(f"Invalid size or alignment for {region.name}")
    first = handoff.regions[0].name
    best = None
    for order in permutations(handoff.regions):
        placement = _first_fit(handoff, order)
        if placement is None:
            continue
        high_water = max(placement[r.name] + r.size_bytes for r in handoff.regions)
        key = (high_water, placement[first], tuple(placement[r.name] for r in handoff.regions))
        if best is None or key < best[0]:
            best = (key, placement)
    if best is None:
        raise ValueError("No optimal physical handoff placement")
    (high_water, _, _), placement = best
    replay(handoff, placement)
    return {
        "schema": "qwen3-residency-placement-v79",
        "status": "OPTIMAL",
        "donor": {"name": handoff.donor_name, "offset_bytes": handoff.donor_offset_bytes,
                  "size_bytes": handoff.donor_bytes, "release": handoff.donor_release},
        "regions": {r.name: {**asdict(r), "offset_bytes": placement[r.name]}
                    for r in handoff.regions},
        "timeline": handoff.timeline,
        "recipient_high_water_bytes": high_water,
        "objective": "Minimum recipient address high-water, then first recipient offset",
    }


def main():
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--out", type=Path, required=True)
    parser.add_argument("--phase", choices=HANDOFFS)
    args = parser.parse_args()
    args.out.mkdir(parents=True, exist_ok=False)
    for phase in (args.phase,) if args.phase else HANDOFFS:
        with (args.out / f"{phase}.json").open("x", encoding="utf-8") as stream:
            json.dump(solve(HANDOFFS[phase]), stream, indent=2)
            stream.write("\n")


if __name__ == "__main__":
    main()

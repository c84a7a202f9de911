"""Where inside a released shared-memory range the epilogue's staging regions go.

The declarative surface is that of ``tilecadence/placement.py`` (``Region`` :13-19, ``Handoff``
:22-28, ``HANDOFFS`` :31-44, ``replay`` :47-62, ``solve`` :65-103, command line :106-115): a *donor*
byte range that a kernel stops reading at a known step of a three-step timeline, and *recipient*
regions (bytes, alignment, half-open live interval in steps) that have to be packed into the donor so
that no two regions that are alive together share a byte. ``solve`` returns the reference's result
dictionary (same keys, same ``schema`` string, same objective text) and ``replay`` raises the same
``ValueError`` messages, so emitted ``placement.json`` files are interchangeable.

Three things differ. The donors describe the sm_100a kernels' shared-memory maps, not the reference's.
There is a second address space: tensor memory (TMEM), 512 columns of 128 lanes x 32 bits per SM, which
holds the score, probability and output tiles of the tcgen05 contractions. A ``TmemMap`` declares those
tiles as regions (columns, column alignment, live interval over the steps of the key loop's steady-state
period, which is cyclic); ``solve_tmem`` packs them with the same rule as the byte tier (regions that are
never alive together may share columns, which is how a probability tile comes to sit in a retired score
buffer) and ``replay_tmem`` checks a column map from first principles.
And the optimum is found by exhaustive search instead of OR-tools CP-SAT: any feasible packing can be
slid towards the donor's start until every region rests against the donor's start or against a region
that is alive with it, without raising the high-water mark or the first region's offset; such
"resting" packings are exactly what placing the regions one after another at the lowest aligned free
address produces, for some order. Trying every order therefore visits an optimal packing.
"""
from __future__ import annotations

import argparse
import itertools
import json
from dataclasses import asdict, dataclass
from pathlib import Path

SCHEMA = "qwen3-residency-placement-v79"
OBJECTIVE = "Minimum recipient address high-water, then first recipient offset"


@dataclass(frozen=True)
class Region:
    """A recipient: ``size_bytes`` at a multiple of ``alignment_bytes``, alive during steps [start, end)."""

    name: str
    size_bytes: int
    alignment_bytes: int
    start: int
    end: int

    def alive_with(self, other: "Region") -> bool:
        return self.start < other.end and other.start < self.end


@dataclass(frozen=True)
class Handoff:
    """A donor range [donor_offset_bytes, +donor_bytes) free from step ``donor_release`` on, and what moves in."""

    donor_name: str
    donor_offset_bytes: int
    donor_bytes: int
    donor_release: int
    regions: tuple[Region, ...]
    timeline: tuple[str, ...]

    @property
    def donor_end(self) -> int:
        return self.donor_offset_bytes + self.donor_bytes


_STEPS_K = ("last_K_read", "K_readers_released_and_epilogue_scatter", "CTA_publish_and_export")
_STEPS_V = ("last_V_read", "V_readers_released_and_epilogue_scatter", "CTA_publish_and_export")

#: The two handoffs of the B200 kernels. Recipient sizes, alignments and live intervals are the
#: reference's; the donors are this build's:
#:   prefill -- stage 0 of the two-stage K ring: 32 KiB at byte 65536 of the CTA's arena, behind the two
#:              32 KiB Q tiles. The ring index is chosen so that the last score MMA always reads stage 0.
#:   decode  -- the V half of stage 0 of the K/V ring: 16 KiB at byte 0. The last tile always lands there.
HANDOFFS = {
    "prefill": Handoff(
        donor_name="terminal_K", donor_offset_bytes=65536, donor_bytes=32768, donor_release=1,
        regions=(Region("head0_lse", 512, 128, start=1, end=3), Region("head1_lse", 512, 128, start=1, end=3)),
        timeline=_STEPS_K),
    "decode": Handoff(
        donor_name="terminal_V", donor_offset_bytes=0, donor_bytes=16384, donor_release=1,
        regions=(Region("output_tile", 2048, 16, start=1, end=3), Region("row_lse", 16, 16, start=1, end=3)),
        timeline=_STEPS_V),
}


def _bytes_collide(first_offset: int, first: Region, second_offset: int, second: Region) -> bool:
    return first_offset < second_offset + second.size_bytes and second_offset < first_offset + first.size_bytes


def replay(handoff: Handoff, offsets: dict[str, int]) -> None:
    """Check a placement from first principles; raises ``ValueError`` on the first violated rule."""
    last_step = len(handoff.timeline)
    checked: list[Region] = []
    for region in handoff.regions:
        offset = offsets[region.name]
        in_time = handoff.donor_release <= region.start < region.end <= last_step
        in_donor = (handoff.donor_offset_bytes <= offset and region.size_bytes > 0
                    and offset + region.size_bytes <= handoff.donor_end)
        aligned = offset % region.alignment_bytes == 0
        if not (in_time and in_donor and aligned):
            raise ValueError(f"Invalid time/address placement for {region.name}")
        for earlier in checked:
            if region.alive_with(earlier) and _bytes_collide(offset, region, offsets[earlier.name], earlier):
                raise ValueError(f"Live byte ranges overlap for {region.name} and {earlier.name}")
        checked.append(region)


def _lowest_free_offset(handoff: Handoff, region: Region, taken: dict[str, int], by_name: dict[str, Region]) -> int:
    """Lowest aligned offset in the donor at which ``region`` collides with nothing already placed."""
    step = region.alignment_bytes
    offset = (handoff.donor_offset_bytes + step - 1) // step * step
    while True:
        blockers = [taken[name] + by_name[name].size_bytes for name in taken
                    if region.alive_with(by_name[name]) and _bytes_collide(offset, region, taken[name], by_name[name])]
        if not blockers:
            return offset
        offset = (max(blockers) + step - 1) // step * step


def _pack_in_order(handoff: Handoff, order, by_name: dict[str, Region]):
    taken: dict[str, int] = {}
    for region in order:
        offset = _lowest_free_offset(handoff, region, taken, by_name)
        if offset + region.size_bytes > handoff.donor_end:
            return None
        taken[region.name] = offset
    return taken


def solve(handoff: Handoff) -> dict:
    """Optimal placement: least recipient high-water mark, ties broken by the first region's offset."""
    regions = handoff.regions
    for region in regions:
        if region.size_bytes <= 0 or region.alignment_bytes <= 0:
            raise ValueError(f"Invalid size or alignment for {region.name}")
    by_name = {region.name: region for region in regions}

    def rank(candidate: dict[str, int]):
        high_water = max(candidate[r.name] + r.size_bytes for r in regions)
        return high_water, candidate[regions[0].name], [candidate[r.name] for r in regions]

    packings = (_pack_in_order(handoff, order, by_name) for order in itertools.permutations(regions))
    feasible = [packing for packing in packings if packing is not None]
    if not feasible:
        raise ValueError("No optimal physical handoff placement")
    chosen = min(feasible, key=rank)
    replay(handoff, chosen)
    placed_regions = {}
    for region in regions:
        record = asdict(region)
        record["offset_bytes"] = chosen[region.name]
        placed_regions[region.name] = record
    return {
        "schema": SCHEMA,
        "status": "OPTIMAL",
        "donor": {"name": handoff.donor_name, "offset_bytes": handoff.donor_offset_bytes,
                  "size_bytes": handoff.donor_bytes, "release": handoff.donor_release},
        "regions": placed_regions,
        "timeline": handoff.timeline,
        "recipient_high_water_bytes": rank(chosen)[0],
        "objective": OBJECTIVE,
    }


# ----------------------------------------------------------------------------------- tensor memory
TMEM_SCHEMA = "b200-tmem-placement-v1"
TMEM_OBJECTIVE = "Minimum column high-water, then first region offset"
TMEM_COLUMNS = 512          # per SM: 128 lanes x 512 columns x 32 bits
TMEM_MIN_ALLOCATION = 32    # tcgen05.alloc hands out a power of two of at least 32 columns


@dataclass(frozen=True)
class TmemRegion:
    """A tile in tensor memory: ``columns`` 32-bit columns (all 128 lanes) at a multiple of
    ``alignment_columns``, alive during steps [start, end) of the map's timeline. With a cyclic timeline
    ``end`` may exceed the period: the region then stays alive into the next round of the loop. ``pipeline``
    names the software pipeline the tile belongs to when a kernel runs several that do not wait for each other
    (the two heads of the prefill kernel): steps of different pipelines cannot be compared, so their tiles
    never share columns."""

    name: str
    columns: int
    alignment_columns: int
    start: int
    end: int
    pipeline: str = ""  # tiles of different (named) pipelines run unsynchronised: they are always alive together


@dataclass(frozen=True)
class TmemMap:
    """The tensor-memory tiles of one kernel. ``timeline`` names the steps; ``cyclic`` says that they are
    the steady-state period of a software-pipelined loop, so that step len(timeline) is step 0 again."""

    name: str
    regions: tuple[TmemRegion, ...]
    timeline: tuple[str, ...]
    cyclic: bool = True
    capacity_columns: int = TMEM_COLUMNS

    def alive_together(self, first: TmemRegion, second: TmemRegion) -> bool:
        if first.pipeline and second.pipeline and first.pipeline != second.pipeline:
            return True
        shifts = (-len(self.timeline), 0, len(self.timeline)) if self.cyclic else (0,)
        return any(first.start < second.end + shift and second.start + shift < first.end for shift in shifts)


#: Tensor-memory tiles of the prefill kernel, one 128-row query tile of two heads per CTA. Steady state of
#: the key loop, one period = one key tile of both heads:
#:   step 0  the score MMA of head 0 fills a score buffer and head 0's softmax warpgroup pulls it
#:   step 1  the same for head 1, while head 0 exponentiates
#: A score buffer is dead as soon as it has been pulled into registers, so the two heads' buffers are never
#: alive together and may share columns. A probability tile P (BF16 pairs: 64 columns for 128 keys) is written
#: after the pull and read by the PV MMA until the head's next pull, and the output accumulators live through
#: the whole loop: neither can share with anything. The solved map is S (shared) | P0 P1 | O0 O1 = all 512
#: columns.
TMEM_MAPS = {
    "prefill": TmemMap(
        name="prefill_two_heads_shared_score",
        regions=(TmemRegion("score_head0", 128, 32, start=0, end=1), TmemRegion("score_head1", 128, 32, start=1, end=2),
                 TmemRegion("probability_head0", 64, 16, start=0, end=2),
                 TmemRegion("probability_head1", 64, 16, start=0, end=2),
                 TmemRegion("output_head0", 128, 32, start=0, end=2), TmemRegion("output_head1", 128, 32, start=0, end=2)),
        timeline=("score_and_pull_head0", "score_and_pull_head1")),
    # Candidate layouts that the planner can price without a kernel being kept for them.
    # Every head a pipeline of its own (one MMA issuer per head, nobody waits for the other head): a head's
    # probabilities are stored over its own retired score buffer, S0/P0 | S1/P1 | O0 | O1. Built and measured:
    # correct, but the head's chain exp -> PV -> next score MMA -> pull is then serial, and one key tile of both
    # heads took 4150 cycles against 3320 with the shared score buffer, whose score MMA runs under the other
    # head's exponentials.
    "prefill_private_scores": TmemMap(
        name="prefill_two_heads_private_scores",
        regions=(TmemRegion("score_head0", 128, 32, start=0, end=1, pipeline="head0"),
                 TmemRegion("score_head1", 128, 32, start=0, end=1, pipeline="head1"),
                 TmemRegion("probability_head0", 64, 16, start=1, end=3, pipeline="head0"),
                 TmemRegion("probability_head1", 64, 16, start=1, end=3, pipeline="head1"),
                 TmemRegion("output_head0", 128, 32, start=0, end=3, pipeline="head0"),
                 TmemRegion("output_head1", 128, 32, start=0, end=3, pipeline="head1")),
        timeline=("score_and_pull", "exponentiate", "pv")),
    # One head per CTA, three score/probability buffers in rotation and one output accumulator.
    "prefill_one_head": TmemMap(
        name="prefill_one_head_three_buffers",
        regions=(TmemRegion("score_a", 128, 32, start=0, end=1), TmemRegion("probability_a", 64, 16, start=1, end=3),
                 TmemRegion("score_b", 128, 32, start=1, end=2), TmemRegion("probability_b", 64, 16, start=2, end=4),
                 TmemRegion("score_c", 128, 32, start=2, end=3), TmemRegion("probability_c", 64, 16, start=0, end=2),
                 TmemRegion("output", 128, 32, start=0, end=3)),
        timeline=("tile_a", "tile_b", "tile_c")),
}


def replay_tmem(tmem_map: TmemMap, columns: dict[str, int]) -> None:
    """Check a column map from first principles; raises ``ValueError`` on the first violated rule."""
    period = len(tmem_map.timeline)
    checked: list[TmemRegion] = []
    for region in tmem_map.regions:
        offset = columns[region.name]
        in_time = 0 <= region.start < region.end and (region.end - region.start <= period if tmem_map.cyclic
                                                      else region.end <= period) and region.start < period
        in_space = offset >= 0 and region.columns > 0 and offset + region.columns <= tmem_map.capacity_columns
        aligned = region.alignment_columns > 0 and offset % region.alignment_columns == 0
        if not (in_time and in_space and aligned):
            raise ValueError(f"Invalid time/column placement for {region.name}")
        for earlier in checked:
            clash = offset < columns[earlier.name] + earlier.columns and columns[earlier.name] < offset + region.columns
            if clash and tmem_map.alive_together(region, earlier):
                raise ValueError(f"Live column ranges overlap for {region.name} and {earlier.name}")
        checked.append(region)


def solve_tmem(tmem_map: TmemMap) -> dict:
    """Optimal column map: least column high-water mark, ties broken by the first region's offset. Same
    search as :func:`solve`: every order of lowest-free-fit placements."""
    regions = tmem_map.regions
    for region in regions:
        if region.columns <= 0 or region.alignment_columns <= 0:
            raise ValueError(f"Invalid size or alignment for {region.name}")
    by_name = {region.name: region for region in regions}

    def lowest_free(region, taken):
        offset = 0
        while True:
            blockers = [taken[name] + by_name[name].columns for name in taken
                        if offset < taken[name] + by_name[name].columns and taken[name] < offset + region.columns
                        and tmem_map.alive_together(region, by_name[name])]
            if not blockers:
                return offset
            step = region.alignment_columns
            offset = (max(blockers) + step - 1) // step * step

    def pack(order):
        taken: dict[str, int] = {}
        for region in order:
            offset = lowest_free(region, taken)
            if offset + region.columns > tmem_map.capacity_columns:
                return None
            taken[region.name] = offset
        return taken

    def rank(candidate):
        return (max(candidate[r.name] + r.columns for r in regions), candidate[regions[0].name],
                [candidate[r.name] for r in regions])

    feasible = [packing for packing in map(pack, itertools.permutations(regions)) if packing is not None]
    if not feasible:
        raise ValueError(f"No tensor-memory placement within {tmem_map.capacity_columns} columns")
    chosen = min(feasible, key=rank)
    replay_tmem(tmem_map, chosen)
    high_water = rank(chosen)[0]
    allocation = TMEM_MIN_ALLOCATION
    while allocation < high_water:
        allocation *= 2
    placed = {}
    for region in regions:
        record = asdict(region)
        record["offset_columns"] = chosen[region.name]
        placed[region.name] = record
    return {"schema": TMEM_SCHEMA, "status": "OPTIMAL", "map": tmem_map.name, "capacity_columns": tmem_map.capacity_columns,
            "regions": placed, "timeline": tmem_map.timeline, "cyclic": tmem_map.cyclic,
            "high_water_columns": high_water, "allocation_columns": allocation, "objective": TMEM_OBJECTIVE}


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--out", required=True, type=Path, help="directory to create; receives <phase>.json")
    parser.add_argument("--phase", choices=sorted(HANDOFFS), help="only this handoff (default: all)")
    arguments = parser.parse_args(argv)
    arguments.out.mkdir(parents=True, exist_ok=False)
    for phase in ([arguments.phase] if arguments.phase else list(HANDOFFS)):
        text = json.dumps(solve(HANDOFFS[phase]), indent=2) + "\n"
        with (arguments.out / f"{phase}.json").open("x", encoding="utf-8") as stream:
            stream.write(text)
        if phase in TMEM_MAPS:
            with (arguments.out / f"{phase}.tmem.json").open("x", encoding="utf-8") as stream:
                stream.write(json.dumps(solve_tmem(TMEM_MAPS[phase]), indent=2) + "\n")


if __name__ == "__main__":
    main()

"""Independent checker and brute-force optimum for the handoff planner. TEST INFRASTRUCTURE ONLY.

``check`` restates ``tilecadence/placement.py:47-62`` (``replay``) on plain tuples so that it
shares no code with the package's planner. ``brute_force`` states the optimisation problem of
``tilecadence/placement.py:65-103`` directly: every aligned slot of every region is tried, pairs
that are live together must not share a byte, and the objective is
``(donor_hi + 1) * high_water + offset(first region)`` (:86), the scalarised form of "minimum
high-water, then minimum first offset". It is exponential and meant for the small declared
handoffs and for small random ones.

Pinned by the reference's known answers, which are the defaults of its own templates
(``cuda/prefill/config.cuh:10-11``: 65536 / 66048; ``cuda/decode/config.cuh:12-13``: 0 / 2048)
and by the behaviour ``tests/test_operator.py:9-19`` asserts (equal offsets raise "overlap").
"""
from itertools import product


def check(donor_offset, donor_bytes, donor_release, steps, regions, offsets):
    """regions: (name, size, alignment, start, end). Raises ValueError like the reference."""
    donor_hi = donor_offset + donor_bytes
    for index, (name, size, alignment, start, end) in enumerate(regions):
        lo = offsets[name]
        hi = lo + size
        if not (donor_release <= start < end <= steps and donor_offset <= lo < hi <= donor_hi
                and lo % alignment == 0):
            raise ValueError(f"Invalid time/address placement for {name}")
        for other_name, other_size, _, other_start, other_end in regions[:index]:
            if max(start, other_start) < min(end, other_end):
                other_lo = offsets[other_name]
                if max(lo, other_lo) < min(hi, other_lo + other_size):
                    raise ValueError(f"Live byte ranges overlap for {name} and {other_name}")


def brute_force(donor_offset, donor_bytes, donor_release, steps, regions):
    """Optimal {name: offset}, high-water and objective value, or None if infeasible."""
    donor_hi = donor_offset + donor_bytes
    choices = []
    for name, size, alignment, start, end in regions:
        first = -(-donor_offset // alignment)
        last = (donor_hi - size) // alignment
        choices.append([slot * alignment for slot in range(first, last + 1)])
    best = None
    for combination in product(*choices):
        offsets = {region[0]: offset for region, offset in zip(regions, combination)}
        try:
            check(donor_offset, donor_bytes, donor_release, steps, regions, offsets)
        except ValueError:
            continue
        high_water = max(offset + region[1] for region, offset in zip(regions, combination))
        objective = (donor_hi + 1) * high_water + combination[0]
        if best is None or objective < best[2]:
            best = (offsets, high_water, objective)
    return best

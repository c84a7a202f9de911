"""Planner: known answers, the reference's replay behaviour, and optimality against brute force.

Follows the assertions of the reference's ``tests/test_operator.py:9-19`` and the known answers
that are the defaults of its templates (``cuda/prefill/config.cuh:10-11``,
``cuda/decode/config.cuh:12-13``).
"""
import random

import pytest

from oracle import placement_oracle
from tilecadence_b200.placement import HANDOFFS, Handoff, Region, replay, solve


def as_tuples(handoff):
    return [(r.name, r.size_bytes, r.alignment_bytes, r.start, r.end) for r in handoff.regions]


def oracle_args(handoff):
    return (handoff.donor_offset_bytes, handoff.donor_bytes, handoff.donor_release, len(handoff.timeline),
            as_tuples(handoff))


def test_known_answers():
    prefill = solve(HANDOFFS["prefill"])
    assert {k: v["offset_bytes"] for k, v in prefill["regions"].items()} == {"head0_lse": 65536, "head1_lse": 66048}
    assert prefill["recipient_high_water_bytes"] == 66560
    decode = solve(HANDOFFS["decode"])
    assert {k: v["offset_bytes"] for k, v in decode["regions"].items()} == {"output_tile": 0, "row_lse": 2048}
    assert decode["recipient_high_water_bytes"] == 2064
    for result in (prefill, decode):
        assert result["schema"] == "qwen3-residency-placement-v79" and result["status"] == "OPTIMAL"
        assert set(result) == {"schema", "status", "donor", "regions", "timeline", "recipient_high_water_bytes",
                               "objective"}


@pytest.mark.parametrize("phase", ("prefill", "decode"))
def test_replay_rejects_overlap_misalignment_and_escape(phase):
    handoff = HANDOFFS[phase]
    offsets = {k: v["offset_bytes"] for k, v in solve(handoff)["regions"].items()}
    replay(handoff, offsets)
    placement_oracle.check(*oracle_args(handoff), offsets)
    first, second = offsets
    clash = dict(offsets)
    clash[second] = clash[first]
    with pytest.raises(ValueError, match="overlap"):
        replay(handoff, clash)
    with pytest.raises(ValueError, match="overlap"):
        placement_oracle.check(*oracle_args(handoff), clash)
    skewed = dict(offsets)
    skewed[second] += 4
    with pytest.raises(ValueError, match="Invalid time/address"):
        replay(handoff, skewed)
    outside = dict(offsets)
    outside[first] = handoff.donor_offset_bytes + handoff.donor_bytes
    with pytest.raises(ValueError, match="Invalid time/address"):
        replay(handoff, outside)


def test_replay_rejects_regions_live_before_release():
    handoff = Handoff("d", 0, 1024, 2, (Region("early", 64, 16, 1, 3),), ("a", "b", "c"))
    with pytest.raises(ValueError, match="Invalid time/address"):
        replay(handoff, {"early": 0})


def test_solver_matches_brute_force_on_random_handoffs():
    rng = random.Random(20240521)
    for _ in range(60):
        steps = rng.randint(2, 5)
        release = rng.randint(0, 1)
        donor_offset = rng.choice((0, 48, 128, 1000))
        regions = []
        for index in range(rng.randint(1, 3)):
            start = rng.randint(release, steps - 1)
            regions.append(Region(f"r{index}", rng.choice((16, 48, 64, 100, 256)), rng.choice((16, 32, 128)),
                                  start, rng.randint(start + 1, steps)))
        handoff = Handoff("donor", donor_offset, rng.choice((256, 384, 512)), release, tuple(regions),
                          tuple(f"s{i}" for i in range(steps)))
        expected = placement_oracle.brute_force(*oracle_args(handoff))
        if expected is None:
            with pytest.raises(ValueError, match="No optimal"):
                solve(handoff)
            continue
        result = solve(handoff)
        offsets = {k: v["offset_bytes"] for k, v in result["regions"].items()}
        placement_oracle.check(*oracle_args(handoff), offsets)
        donor_hi = handoff.donor_offset_bytes + handoff.donor_bytes
        objective = (donor_hi + 1) * result["recipient_high_water_bytes"] + offsets[regions[0].name]
        assert objective == expected[2], (handoff, offsets, expected)


def test_time_disjoint_regions_may_share_bytes():
    handoff = Handoff("d", 0, 256, 0, (Region("a", 256, 16, 0, 1), Region("b", 256, 16, 1, 2)), ("x", "y"))
    result = solve(handoff)
    assert result["regions"]["a"]["offset_bytes"] == result["regions"]["b"]["offset_bytes"] == 0

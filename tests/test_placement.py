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


# ----------------------------------------------------------------------------------- tensor memory tier
from tilecadence_b200.placement import TMEM_MAPS, TmemMap, TmemRegion, replay_tmem, solve_tmem  # noqa: E402


def tmem_brute_force(tmem_map):
    """Every aligned column of every region; the least (high-water, first offset) that ``replay_tmem`` accepts."""
    from itertools import product

    choices = [range(0, tmem_map.capacity_columns - r.columns + 1, r.alignment_columns) for r in tmem_map.regions]
    best = None
    for combination in product(*choices):
        columns = {r.name: c for r, c in zip(tmem_map.regions, combination)}
        try:
            replay_tmem(tmem_map, columns)
        except ValueError:
            continue
        key = (max(c + r.columns for r, c in zip(tmem_map.regions, combination)), combination[0])
        if best is None or key < best:
            best = key
    return best


def test_prefill_tensor_memory_map_is_the_kernels_layout():
    """Scores of the two heads share one buffer (never alive together); P and O tiles fill the rest: all 512."""
    solved = solve_tmem(TMEM_MAPS["prefill"])
    assert {k: v["offset_columns"] for k, v in solved["regions"].items()} == {
        "score_head0": 0, "score_head1": 0, "probability_head0": 128, "probability_head1": 192,
        "output_head0": 256, "output_head1": 384}
    # the measured alternative: the heads' pipelines are not synchronised, so nothing of one head shares columns
    # with anything of the other, and a head's probabilities sit over its own retired score buffer
    private = solve_tmem(TMEM_MAPS["prefill_private_scores"])
    assert {k: v["offset_columns"] for k, v in private["regions"].items()} == {
        "score_head0": 0, "score_head1": 128, "probability_head0": 0, "probability_head1": 128,
        "output_head0": 256, "output_head1": 384}
    assert solved["high_water_columns"] == 512 and solved["allocation_columns"] == 512
    assert solved["schema"] == "b200-tmem-placement-v1" and solved["status"] == "OPTIMAL"


def test_candidate_tensor_memory_maps_fit_and_reuse_retired_score_buffers():
    for name in ("prefill_private_scores", "prefill_one_head"):
        tmem_map = TMEM_MAPS[name]
        solved = solve_tmem(tmem_map)
        columns = {k: v["offset_columns"] for k, v in solved["regions"].items()}
        replay_tmem(tmem_map, columns)
        assert solved["high_water_columns"] <= 512 and solved["allocation_columns"] == 512
        total = sum(r.columns for r in tmem_map.regions)
        assert total > 512 >= solved["high_water_columns"]  # only possible because dead tiles give up their columns
    # a probability tile sits in the columns of its own retired score buffer
    private = {k: v["offset_columns"] for k, v in solve_tmem(TMEM_MAPS["prefill_private_scores"])["regions"].items()}
    assert private["probability_head0"] == private["score_head0"] and private["probability_head1"] == private["score_head1"]


def test_tensor_memory_replay_rejects_overlap_misalignment_and_overflow():
    tmem_map = TMEM_MAPS["prefill"]
    columns = {k: v["offset_columns"] for k, v in solve_tmem(tmem_map)["regions"].items()}
    replay_tmem(tmem_map, columns)
    clash = dict(columns, probability_head1=columns["probability_head0"])
    with pytest.raises(ValueError, match="Live column ranges overlap"):
        replay_tmem(tmem_map, clash)
    skewed = dict(columns, output_head1=columns["output_head1"] - 8)
    with pytest.raises(ValueError, match="Invalid time/column"):
        replay_tmem(tmem_map, skewed)
    outside = dict(columns, output_head1=448)
    with pytest.raises(ValueError, match="Invalid time/column"):
        replay_tmem(tmem_map, outside)
    # the shared score buffer is legal only because the two heads' scores are never alive together
    both_alive = TmemMap("x", tuple(TmemRegion(r.name, r.columns, r.alignment_columns, 0, 2) for r in tmem_map.regions),
                         tmem_map.timeline)
    with pytest.raises(ValueError, match="Live column ranges overlap"):
        replay_tmem(both_alive, columns)
    with pytest.raises(ValueError, match="No tensor-memory placement"):
        solve_tmem(both_alive)  # 640 columns alive at once


def test_tensor_memory_solver_is_optimal_on_small_random_maps():
    rng = random.Random(7)
    for _ in range(40):
        period = rng.randint(2, 4)
        regions = []
        for index in range(rng.randint(2, 4)):
            start = rng.randrange(period)
            regions.append(TmemRegion(f"r{index}", rng.choice((16, 32, 64)), rng.choice((16, 32)), start,
                                      start + rng.randint(1, period)))
        tmem_map = TmemMap("random", tuple(regions), tuple(f"s{i}" for i in range(period)), cyclic=True,
                           capacity_columns=128)
        want = tmem_brute_force(tmem_map)
        if want is None:
            with pytest.raises(ValueError):
                solve_tmem(tmem_map)
            continue
        solved = solve_tmem(tmem_map)
        got = (solved["high_water_columns"], solved["regions"]["r0"]["offset_columns"])
        assert got == want


def test_cyclic_lifetimes_wrap_around_the_period():
    steps = ("a", "b", "c")
    late = TmemRegion("late", 64, 32, start=2, end=4)     # alive in step c and in step a of the next round
    first = TmemRegion("first", 64, 32, start=0, end=1)   # alive in step a: collides with `late`
    middle = TmemRegion("middle", 64, 32, start=1, end=2)  # alive in step b only: may share with both
    solved = solve_tmem(TmemMap("wrap", (late, first, middle), steps, cyclic=True, capacity_columns=128))
    columns = {k: v["offset_columns"] for k, v in solved["regions"].items()}
    assert columns["late"] != columns["first"] and solved["high_water_columns"] == 128
    assert columns["middle"] in (columns["late"], columns["first"])
    straight = solve_tmem(TmemMap("no-wrap", (TmemRegion("late", 64, 32, 2, 3), first, middle), steps, cyclic=False,
                                  capacity_columns=128))
    assert straight["high_water_columns"] == 64

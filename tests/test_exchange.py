"""CPU regressions for the shared residency exchange planner and its CUDA lowering.

Follows the reference's ``tests/test_exchange.py`` (checkpoint frontier :17-59, residency exchange
:62-138), with the emitted-text assertions adapted to the sm_100a primitive names, and pins the
verifier and the lowering oracle to outputs of the reference's own ``exchange.verify`` and
``model.lowering_trace`` (``tests/golden/exchange_golden.json``).
"""
from copy import deepcopy
import json
from pathlib import Path
import re
import subprocess
import sys
from types import SimpleNamespace

import pytest

from tilecadence_b200 import emit_exchange as emitter
from tilecadence_b200 import exchange, model

GOLDEN = json.loads((Path(__file__).parent / "golden" / "exchange_golden.json").read_text())


def span(copy):
    return copy["offset_bytes"], copy["offset_bytes"] + copy["occupied_bytes"]


def test_checkpoint_barriers_neither_complete_async_copies_nor_hide_old_reads():
    frontier = GOLDEN["frontier"]
    problem = SimpleNamespace(provenance=frontier["provenance"])
    rows = model.lowering_trace(problem, frontier["record"])
    assert rows == frontier["reference_trace"]
    trace = {row["id"]: row for row in rows}
    assert trace["store_p"]["shared_read_write_hazards"] == [["store_p", "issue_q"]]
    assert trace["store_p"]["read_mask_after"] == 0
    assert trace["read_p"]["read_mask_after"] == 1
    assert trace["read_p"]["issued_groups_after"] == 2 and trace["read_p"]["ready_groups_after"] == 1
    assert trace["read_v"]["wait_before_load"] and not trace["read_v_again"]["wait_before_load"]
    assert trace["issue_k"]["read_mask_before"] == 17
    assert trace["issue_k"]["shared_read_write_hazards"] == [["issue_k", "store_p"]]
    assert trace["issue_k"]["release_before_write"]


@pytest.fixture(scope="module", params=exchange.ARMS)
def solved(request):
    problem = exchange.build_problem(request.param)
    result = model.solve(problem, max_time_seconds=2)
    assert result["status"] in ("FEASIBLE", "OPTIMAL")
    return request.param, problem, result


def test_plans_are_deterministic_and_match_the_reference_verifier(solved):
    arm, problem, result = solved
    golden = GOLDEN["arms"][arm]
    assert result["events"] == golden["plan"]["events"] and result["copies"] == golden["plan"]["copies"]
    certificate = exchange.verify(exchange.build_contract(arm), result)
    reference = golden["reference_certificate"]
    assert {k: v for k, v in certificate.items() if k != "scope"} == {k: v for k, v in reference.items() if k != "scope"}
    assert result["lowering_trace"] == golden["reference_trace"]
    assert result["replay"]["residency_certificate"] == certificate
    assert result["objective"] == 128 * len(result["events"]) + result["source_features"]["rf_kib_steps"]


def test_plans_are_accepted_by_the_reference_replay(solved):
    """The reference's full ``model.replay`` (model.py:1205-1355) accepted each of these plans for its own
    problem of the arm and reported the quantities stored in the fixture; this package's replay reports
    the same ones for the same plan."""
    arm, problem, result = solved
    theirs = GOLDEN["arms"][arm]["reference_replay"]
    ours = result["replay"]
    assert theirs["valid"] is True and ours["valid"] is True
    for key in ("peak_bytes", "executions", "q_global_loads", "source_order_steps", "objective", "objective_unit",
                "objective_features"):
        assert ours[key] == theirs[key], key
    assert theirs["pure_p_recoveries"] == 0 and theirs["recomputations"] == {} and theirs["control_storage_bytes"] == 0
    without_scope = lambda certificate: {k: v for k, v in certificate.items() if k != "scope"}  # a free-text note
    assert without_scope(theirs["residency_exchange_v78"]) == without_scope(ours["residency_certificate"])
    assert theirs["output_states"] == result["output_states"]
    # the fields the reference's replay reads beyond events and copies
    assert set(result) >= {"profiles", "best_bound", "lexicographic_objective", "objective_features",
                           "cp_source_features", "model_sha256", "optimality_certified", "actions"}
    assert all({"profile_key", "profile_cost"} <= set(event) for event in result["events"])
    assert result["best_bound"] <= result["objective"]
    assert result["optimality_certified"] == (result["best_bound"] == result["objective"]) == (result["status"] == "OPTIMAL")
    assert len(result["model_sha256"]) == 64


def test_reference_plan_fields_are_enough_for_the_verifier():
    """The verifier needs nothing but events and copies: it accepts the stored golden plan as is."""
    for arm, golden in GOLDEN["arms"].items():
        exchange.verify(exchange.build_contract(arm), golden["plan"])


def test_verifier_refuses_a_plan_that_recomputes_probabilities():
    """``P recomputation is excluded`` (reference exchange.py:186): a ``recover_p`` event voids the certificate."""
    plan = deepcopy(GOLDEN["arms"]["one"]["plan"])
    extra = deepcopy(plan["events"][-1])
    extra.update(id="recover_P0#0", kind="recover_p", start=extra["end"], end=extra["end"] + 1)
    plan["events"].append(extra)
    with pytest.raises(ValueError, match="P recomputation is excluded"):
        exchange.verify(exchange.build_contract("one"), plan)


@pytest.fixture(scope="module")
def two_checkpoints():
    problem = exchange.build_problem("relocated_two_p")
    result = model.solve(problem, max_time_seconds=2)
    return (problem, result, {c["id"]: c for c in result["copies"]}, {e["id"]: e for e in result["events"]},
            {row["id"]: row for row in result["lowering_trace"]})


def test_disjoint_probability_checkpoints_reuse_the_live_donors_range(two_checkpoints):
    _, _, copies, events, _ = two_checkpoints
    donor, restored = copies["copy_Q#0:out0"], copies["copy_Q#1:out0"]
    p0, p1 = copies["store_P0#0:out0"], copies["store_P1#0:out0"]
    (donor_lo, donor_hi), (restore_lo, restore_hi) = span(donor), span(restored)
    assert restore_hi <= donor_lo or donor_hi <= restore_lo
    assert donor["end"] <= p0["start"]
    assert p0["available"] <= restored["start"]
    assert restored["end"] <= p1["start"]
    assert p1["available"] < min(p0["end"], p1["end"])
    spans = sorted([span(p0), span(p1)])
    assert spans[0][1] <= spans[1][0]
    for lo, hi in spans:
        assert donor_lo <= lo and hi <= donor_hi and hi - lo == 4096
    assert events["load_Q#0"]["inputs"] == [donor["id"]]
    assert events["load_Q#1"]["inputs"] == [restored["id"]]
    assert "load_Q#0:out0" in events["qk_0#0"]["inputs"] and "load_Q#1:out0" in events["qk_1#0"]["inputs"]
    for tile, checkpoint in enumerate((p0, p1)):
        assert events[f"load_P{tile}#0"]["inputs"] == [checkpoint["id"]]
        assert f"load_P{tile}#0:out0" in events[f"pv_{tile}_1#0"]["inputs"]


def test_lowering_keeps_checkpoint_barriers_separate_from_copy_acquire(two_checkpoints):
    problem, result, copies, _, trace = two_checkpoints
    for tile in (0, 1):
        store, load = trace[f"store_P{tile}#0"], trace[f"load_P{tile}#0"]
        bit = 1 << (copies[f"store_P{tile}#0:out0"]["offset_bytes"] // 4096)
        for row in (store, load):
            assert row["ready_cutoff_before"] == row["ready_cutoff_after"]
            assert row["ready_groups_before"] == row["ready_groups_after"]
            assert row["issued_groups_before"] == row["issued_groups_after"]
            assert not row["wait_before_load"]
        assert store["read_mask_after"] == 0
        assert load["read_mask_after"] == load["read_mask_before"] | bit
    source, manifest = emitter.source_for(problem, result)
    assert source.count("issue_g2s<Element,64,128,") == 2
    assert source.count("store_checkpoint(") == 2
    assert source.count("load_checkpoint<Element>(") == 2
    assert manifest["source_ready_mask_certificate"] == result["lowering_trace"]
    lines = source.splitlines()
    for tile in (0, 1):
        bounds = manifest["event_source_lines"][f"load_P{tile}#0"]
        body = "\n".join(lines[bounds["comment_line"] - 1:bounds["last_line"]])
        match = re.search(r"load_checkpoint<Element>\((s\d+),ctx\)", body)
        assert match is not None
        address = copies[f"store_P{tile}#0:out0"]["offset_bytes"]
        assert f"Element* {match[1]}=reinterpret_cast<Element*>(arena+{address});" in source
    waits = sum(row["wait_before_load"] for row in result["lowering_trace"])
    assert source.count("acquire_copies<") == waits == result["source_features"]["consumer_wait_count"]
    assert source.count("release_shared_reads();") == sum(row["release_before_write"] for row in result["lowering_trace"])
    assert result["source_features"]["release_barrier_count"] == sum(
        row["release_before_write"] for row in result["lowering_trace"] if row["kind"] in ("copy_g2s", "normalize_store"))


def test_replay_rejects_tampering(two_checkpoints):
    problem, result, copies, _, _ = two_checkpoints
    tampered = deepcopy(result)
    load = next(row for row in tampered["lowering_trace"] if row["id"] == "load_P0#0")
    load["read_mask_after"] &= ~(1 << (copies["store_P0#0:out0"]["offset_bytes"] // 4096))
    with pytest.raises(ValueError, match="lowering trace"):
        model.replay(problem, tampered)
    moved = deepcopy(result)
    next(c for c in moved["copies"] if c["id"] == "store_P1#0:out0")["offset_bytes"] = \
        copies["store_P0#0:out0"]["offset_bytes"]
    with pytest.raises(ValueError):
        model.replay(problem, moved)
    swapped = deepcopy(result)
    a, b = swapped["events"][5], swapped["events"][6]
    a["start"], a["end"], b["start"], b["end"] = b["start"], b["end"], a["start"], a["end"]
    with pytest.raises(ValueError):
        model.replay(problem, swapped)
    with pytest.raises(ValueError, match="differs from the frozen arm"):
        exchange.verify({**exchange.build_contract("one"), "arena_slabs": 4}, result)


def test_committed_plan_is_what_the_emitter_produces(two_checkpoints):
    problem, result, _, _, _ = two_checkpoints
    source, _ = emitter.source_for(problem, result)
    committed = Path(emitter.__file__).parent / "csrc" / "exchange" / "plan.cu"
    assert committed.read_text() == source


def test_cli_writes_certificates_sources_and_manifests(tmp_path):
    out = tmp_path / "exchange"
    subprocess.run([sys.executable, "-m", "tilecadence_b200.exchange", "--out", str(out), "--arm", "one", "--arm", "retain",
                    "--seconds", "1"], check=True, cwd=Path(__file__).resolve().parents[1])
    for arm in ("one", "retain"):
        certificate = json.loads((out / arm / "residency_certificate.json").read_text())
        assert certificate["contract"]["arm"] == arm
        emitted = {path.name for path in (out / arm / "emitted").iterdir()}
        assert {"plan.cu", "backend.cuh", "manifest.json", "tc_ptx.cuh", "tc_host.cuh", "tc_abi.cu",
                "tilecadence_b200.h"} <= emitted
        assert (out / arm / "solver" / "result.json").is_file()
    with pytest.raises(subprocess.CalledProcessError):
        subprocess.run([sys.executable, "-m", "tilecadence_b200.exchange", "--out", str(out)], check=True,
                       cwd=Path(__file__).resolve().parents[1], capture_output=True)


def test_problem_round_trips_through_json():
    problem = exchange.build_problem("multi")
    again = model.problem_from_dict(json.loads(json.dumps(model.problem_to_dict(problem))))
    assert model.validate_problem(again)
    assert model.solve(again, max_time_seconds=1)["events"] == model.solve(problem, max_time_seconds=1)["events"]

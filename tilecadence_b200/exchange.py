"""Generate and verify controlled shared-memory residency exchange plans.

Same surface as ``tilecadence/exchange.py``: four arms (``ARMS`` :11, ``RECIPIENTS`` :18), a frozen
contract per arm (``build_contract`` :21-33), ``build_problem`` (:41-63), an independent ``verify``
that re-derives every promise of the contract from a solved plan and returns the residency
certificate (:165-289), and the CLI (:292-321).

The arms differ in what moves into the 16 KiB that the first Q copy vacates after the first QK:
``retain`` keeps Q where it is; ``one`` parks the first probability tile P0 there (a 4 KiB checkpoint)
and re-copies Q elsewhere for the second QK; ``multi`` parks P0 and the V stripe ``V0_1``;
``relocated_two_p`` parks P0 and P1.

The reference states the arm's rules as CP-SAT constraints (``constrain`` :66-162); here they are a
declarative plan (bindings, extra selected actions, ordering pairs, donor/restore/recipient roles)
that :mod:`tilecadence_b200.model` feeds to its branch-and-bound planner.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

from . import model

ARMS = ("retain", "one", "multi", "relocated_two_p")
PROVENANCE_KEY = "residency_exchange_v78"
INITIAL_Q = "copy_Q#0:out0"
RESTORED_Q = "copy_Q#1:out0"
P0 = "store_P0#0:out0"
P1 = "store_P1#0:out0"
V = "copy_V0_1#0:out0"
RECIPIENTS = {"retain": (), "one": (P0,), "multi": (P0, V), "relocated_two_p": (P0, P1)}


def build_contract(arm):
    model.require(arm in ARMS, f"Unknown residency arm: {arm}")
    return {
        "revision": "v78",
        "arm": arm,
        "arena_slabs": 8,
        "slab_bytes": model.SLAB_BYTES,
        "donor": INITIAL_Q,
        "restore": RESTORED_Q if arm != "retain" else None,
        "recipients": list(RECIPIENTS[arm]),
        "scope": "M64/N64/D128 split-V, shared128 output, exact two QK, no P rematerialization",
    }


def _arm(contract):
    arm = contract.get("arm")
    model.require(contract == build_contract(arm), "Residency contract differs from the frozen arm")
    return arm


def plan_for(arm):
    """The arm's rules as data for the planner (what ``constrain`` adds to the reference's CP model)."""
    contract = build_contract(arm)
    plan = {"contract": contract, "arm": arm, "donor": INITIAL_Q, "restore": contract["restore"],
            "recipients": list(RECIPIENTS[arm]), "selected": [], "before": [], "window_open": [],
            "bindings": {"load_Q#0": {"0": INITIAL_Q}, "qk_0#0": {"0": "load_Q#0:out0"}}}
    if arm == "retain":
        # The second QK may reuse the first register copy of Q or load it again from the one shared copy.
        plan["alternatives"] = [{"qk_1#0:0": "load_Q#0:out0"},
                                {"qk_1#0:0": "load_Q#1:out0", "load_Q#1:0": INITIAL_Q}]
        return plan
    bindings, before = plan["bindings"], plan["before"]
    bindings["load_Q#1"] = {"0": RESTORED_Q}
    bindings["qk_1#0"] = {"0": "load_Q#1:out0"}
    before.append(["qk_0#0", "copy_Q#1"])

    def checkpoint(tile, port):
        produced = f"stats_{tile}#0:out{port}"
        bindings[f"store_P{tile}#0"] = {"0": produced}
        bindings[f"load_P{tile}#0"] = {"0": f"store_P{tile}#0:out0"}
        bindings[f"pv_{tile}_0#0"] = {"0": produced}
        bindings[f"pv_{tile}_1#0"] = {"0": f"load_P{tile}#0:out0"}
        before.append([f"pv_{tile}_0#0", f"load_P{tile}#0"])

    checkpoint(0, 2)
    before += [["pv_0_0#0", "qk_1#0"], ["qk_1#0", "load_P0#0"], ["store_P0#0", "copy_Q#1", 1]]
    plan["window_open"] = [P0]
    if arm == "multi":
        bindings["load_V0_1#0"] = {"0": V}
        bindings["pv_0_1#0"]["1"] = "load_V0_1#0:out0"
        before += [["copy_V0_1#0", "copy_Q#1", 1], ["copy_Q#1", "load_V0_1#0"]]
        plan["window_open"] = [P0, V]
    elif arm == "relocated_two_p":
        checkpoint(1, 3)
        # P1 joins P0 in the donor's range only after Q has been re-copied and re-read elsewhere.
        before += [["store_P1#0", "load_P0#0"], ["load_Q#1", "store_P1#0"]]
    return plan


def build_problem(arm):
    contract = build_contract(arm)
    # Source-level proxies only. Calibrated comparisons require compiled GPU timings.
    objective = {
        "unit": "cost_ticks",
        "constant": 0,
        "terms": [{"feature": "source_actions", "coefficient": 128},
                  {"feature": "rf_kib_steps", "coefficient": 1}],
        "provenance": {"scope": "Same uncalibrated action-count and RF liveness proxy for every arm"},
    }
    return model.build_problem(arena_slabs=contract["arena_slabs"], allow_probability_spill=True,
                               objective_spec=objective, close_workspace_smem_bytes=8192,
                               provenance={PROVENANCE_KEY: contract}, plan=plan_for(arm))


def verify(contract, result):
    """Independently validate actual selected bindings, intervals, and byte ranges."""
    arm = _arm(contract)
    model.require(result.get("status") in ("OPTIMAL", "FEASIBLE"), "Residency verification needs a solved plan")
    events = {row["id"]: row for row in result["events"]}
    copies = {row["id"]: row for row in result["copies"]}
    slab, arena = model.SLAB_BYTES, contract["arena_slabs"] * model.SLAB_BYTES

    def need(condition, message):
        model.require(condition, f"{arm}: {message}")

    def span(copy):
        lo, size = copy["offset_bytes"], copy["occupied_bytes"]
        need(copy["tier"] == "smem" and model.integer(lo) and model.integer(size, 1) and lo % slab == 0
             and size % slab == 0 and lo + size <= arena, f"invalid arena span for {copy['id']}")
        return [lo, lo + size]

    def bound(event, port, source):
        need(event in events and source in copies and events[event]["inputs"][port] == source,
             f"{event} must consume {source} at port {port}")

    def ordered(*names):
        need(all(events[a]["end"] <= events[b]["start"] for a, b in zip(names, names[1:])),
             "required source order " + " < ".join(names) + " is violated")

    need({e["id"] for e in events.values() if e["kind"] == "qk"} == {"qk_0#0", "qk_1#0"}, "exactly one required QK per tile")
    repeats = {"load_Q#1"} | ({"copy_Q#1"} if arm != "retain" else set())
    need(all(i.endswith("#0") or i in repeats for i in events), "unexpected repeated action outside the common graph")
    shared_q = {c["id"] for c in copies.values() if c["tier"] == "smem" and c["role"] == "q"}
    need(shared_q == ({INITIAL_Q} if arm == "retain" else {INITIAL_Q, RESTORED_Q}), "unexpected shared Q copies")
    bound("load_Q#0", 0, INITIAL_Q)
    bound("qk_0#0", 0, "load_Q#0:out0")
    donor = copies[INITIAL_Q]
    donor_span = span(donor)
    need(donor["occupied_bytes"] == 16384, "full Q donor must occupy 16 KiB")
    certificate = {
        "contract": contract,
        "donor_span_bytes": donor_span,
        "original_q_shared_source_steps": [donor["start"], donor["end"]],
        "recipients": [],
        "scope": "Address reservation and source-order dependencies; readiness on the GPU is what the emitted waits enforce",
    }
    checkpoints = {e["id"] + ":out0" for e in events.values() if e["kind"] == "store_r2s"}
    need(checkpoints == {p for p in RECIPIENTS[arm] if p.startswith("store_")}, "unexpected checkpoint path")
    if arm == "retain":
        source = events["qk_1#0"]["inputs"][0]
        if source != "load_Q#0:out0":
            bound("qk_1#0", 0, "load_Q#1:out0")
            bound("load_Q#1", 0, INITIAL_Q)
        certificate["qk1_q_register_source"] = source
        return certificate

    bound("load_Q#1", 0, RESTORED_Q)
    bound("qk_1#0", 0, "load_Q#1:out0")
    restored = copies[RESTORED_Q]
    restore_span = span(restored)
    need(restored["occupied_bytes"] == donor["occupied_bytes"]
         and (restore_span[1] <= donor_span[0] or donor_span[1] <= restore_span[0]),
         "restore Q must use a disjoint address range")
    need(events["qk_0#0"]["end"] <= restored["start"], "restore must follow the original QK")
    need(copies["load_Q#0:out0"]["end"] == events["qk_0#0"]["end"], "original Q RF held beyond first QK")
    certificate["restore_span_bytes"] = restore_span
    certificate["restore_issue_source_step"] = restored["start"]

    def checkpoint(tile, port):
        produced = f"stats_{tile}#0:out{port}"
        bound(f"store_P{tile}#0", 0, produced)
        bound(f"load_P{tile}#0", 0, f"store_P{tile}#0:out0")
        bound(f"pv_{tile}_0#0", 0, produced)
        bound(f"pv_{tile}_1#0", 0, f"load_P{tile}#0:out0")
        ordered(f"pv_{tile}_0#0", f"load_P{tile}#0")

    checkpoint(0, 2)
    ordered("pv_0_0#0", "qk_1#0", "load_P0#0")
    if arm == "multi":
        bound("load_V0_1#0", 0, V)
        bound("pv_0_1#0", 1, "load_V0_1#0:out0")
        ordered("copy_Q#1", "load_V0_1#0")
    elif arm == "relocated_two_p":
        checkpoint(1, 3)
        ordered("store_P1#0", "load_P0#0")

    tenants = [copies[identity] for identity in RECIPIENTS[arm]]
    for copy in tenants:
        lo, hi = span(copy)
        need(donor_span[0] <= lo < hi <= donor_span[1] and hi - lo == slab,
             f"recipient {copy['id']} must occupy one slab in the vacated donor")
        need(donor["end"] <= copy["start"] and copy["available"] < copy["end"],
             f"recipient {copy['id']} has invalid donor reuse or no later consumer")
        certificate["recipients"].append({"copy": copy["id"], "span_bytes": [lo, hi],
                                          "source_steps": [copy["start"], copy["end"]],
                                          "producer_end": copy["available"]})
    early = tenants[:1] if arm == "relocated_two_p" else tenants
    pre_start, pre_end = max(c["available"] for c in early), restored["start"]
    need(pre_start < pre_end <= min(c["end"] for c in early), "no pre-restore recipient window")
    certificate["pre_restore_reservation_source_steps"] = [pre_start, pre_end]
    for copy in copies.values():
        if copy["tier"] != "smem" or copy["id"] in (INITIAL_Q, RESTORED_Q, *RECIPIENTS[arm]):
            continue
        lo, hi = span(copy)
        need(copy["end"] <= pre_start or pre_end <= copy["start"] or hi <= donor_span[0] or donor_span[1] <= lo,
             f"undeclared occupant {copy['id']} in the pre-restore window")
    joint_start, joint_end = max(c["available"] for c in tenants), min(c["end"] for c in tenants)
    need(joint_start < joint_end, "no common recipient reservation window")
    if len(tenants) == 2:
        a, b = (span(c) for c in tenants)
        need(a[1] <= b[0] or b[1] <= a[0], "simultaneous recipients overlap in address")
    if arm == "relocated_two_p":
        need(restored["available"] <= joint_start, "P1 is not available before Q is restored elsewhere")
    certificate["joint_reservation_source_steps"] = [joint_start, joint_end]
    return certificate


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--out", type=Path, required=True)
    parser.add_argument("--arm", action="append", choices=ARMS)
    parser.add_argument("--seconds", type=float, default=15)
    parser.add_argument("--no-emit", action="store_true")
    args = parser.parse_args()
    model.require(0 < args.seconds <= 120, "Per-arm search budget must be between zero and 120 seconds")
    arms = args.arm or ARMS
    model.require(len(set(arms)) == len(arms), "Each arm may only be generated once")
    args.out.mkdir(parents=True, exist_ok=False)
    failures = []
    for arm in arms:
        role = args.out / arm
        role.mkdir()
        problem = build_problem(arm)
        try:
            result = model.solve(problem, max_time_seconds=args.seconds, artifact_dir=role / "solver")
            certificate = verify(problem.provenance[PROVENANCE_KEY], result)
            (role / "residency_certificate.json").write_text(json.dumps(certificate, indent=2) + "\n")
            if not args.no_emit:
                from .emit_exchange import emit

                emit(problem, result, role / "emitted")
            print(f"{arm}: {result['status']}; {result['finish_step']} source steps", flush=True)
        except (ValueError, RuntimeError) as error:
            (role / "failure.txt").write_text(str(error) + "\n")
            failures.append(arm)
            print(f"{arm}: {error}", flush=True)
    if failures:
        raise SystemExit("Unsuccessful arms: " + ", ".join(failures))


if __name__ == "__main__":
    main()

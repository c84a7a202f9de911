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
        # the reference's spelling (exchange.py:47-55), so that serialised problems are interchangeable
        "terms": [{"feature": "source_actions", "coefficient": 128, "match": {}},
                  {"feature": "rf_payload_kib_steps", "coefficient": 1, "source": {"kind": "rf_kib_steps"}}],
        "provenance": {"scope": "Same uncalibrated action-count and RF liveness proxy for every arm"},
    }
    return model.build_problem(arena_slabs=contract["arena_slabs"], allow_probability_spill=True,
                               objective_spec=objective, close_workspace_smem_bytes=8192,
                               provenance={PROVENANCE_KEY: contract}, plan=plan_for(arm))


class _Audit:
    """Read-only view of a solved plan with the checks ``verify`` is built from. Every failed check
    raises ``ValueError`` (through :func:`model.require`) prefixed with the arm's name."""

    def __init__(self, arm, contract, result):
        self.arm = arm
        self.slab = model.SLAB_BYTES
        self.arena_bytes = contract["arena_slabs"] * model.SLAB_BYTES
        self.events = {event["id"]: event for event in result["events"]}
        self.copies = {copy["id"]: copy for copy in result["copies"]}

    def check(self, holds, what):
        model.require(holds, f"{self.arm}: {what}")

    def byte_span(self, copy):
        """[first byte, one past the last byte] of a shared-memory copy, after checking it is slab-shaped."""
        first, length = copy["offset_bytes"], copy["occupied_bytes"]
        well_formed = (copy["tier"] == "smem" and model.integer(first) and model.integer(length, 1)
                       and first % self.slab == 0 and length % self.slab == 0 and first + length <= self.arena_bytes)
        self.check(well_formed, f"invalid arena span for {copy['id']}")
        return [first, first + length]

    def reads(self, consumer, port, producer_output):
        known = consumer in self.events and producer_output in self.copies
        self.check(known and self.events[consumer]["inputs"][port] == producer_output,
                   f"{consumer} must consume {producer_output} at port {port}")

    def in_source_order(self, *names):
        pairs = zip(names, names[1:])
        self.check(all(self.events[first]["end"] <= self.events[second]["start"] for first, second in pairs),
                   "required source order " + " < ".join(names) + " is violated")

    def checkpoint_path(self, tile, stats_port):
        """P of ``tile`` goes registers -> shared -> registers between its two PV stripes."""
        probabilities = f"stats_{tile}#0:out{stats_port}"
        store, load = f"store_P{tile}#0", f"load_P{tile}#0"
        self.reads(store, 0, probabilities)
        self.reads(load, 0, f"{store}:out0")
        self.reads(f"pv_{tile}_0#0", 0, probabilities)
        self.reads(f"pv_{tile}_1#0", 0, f"{load}:out0")
        self.in_source_order(f"pv_{tile}_0#0", load)


def _disjoint(first, second):
    return first[1] <= second[0] or second[1] <= first[0]


def verify(contract, result):
    """Re-derive every promise of the arm's contract from a solved plan's events and copies.

    Returns the residency certificate (donor and restore spans, each recipient's span and source steps,
    the reservation windows); raises ``ValueError`` if the plan breaks the contract. Nothing here trusts
    the planner: only the selected bindings, intervals and byte offsets recorded in ``result`` are read.
    """
    arm = _arm(contract)
    model.require(result.get("status") in ("OPTIMAL", "FEASIBLE"), "Residency verification needs a solved plan")
    audit = _Audit(arm, contract, result)
    events, copies, check = audit.events, audit.copies, audit.check
    moved_in = RECIPIENTS[arm]

    # -- what every arm shares: the action set, the two Q reads, the original Q copy
    score_actions = {event["id"] for event in events.values() if event["kind"] == "qk"}
    check(score_actions == {"qk_0#0", "qk_1#0"}, "exactly one required QK per tile")
    check(not any(event["kind"] == "recover_p" for event in events.values()), "P recomputation is excluded")
    allowed_repeats = {"load_Q#1"} if arm == "retain" else {"load_Q#1", "copy_Q#1"}
    check(all(identity.endswith("#0") or identity in allowed_repeats for identity in events),
          "unexpected repeated action outside the common graph")
    q_in_shared = {copy["id"] for copy in copies.values() if copy["role"] == "q" and copy["tier"] == "smem"}
    check(q_in_shared == ({INITIAL_Q} if arm == "retain" else {INITIAL_Q, RESTORED_Q}), "unexpected shared Q copies")
    audit.reads("load_Q#0", 0, INITIAL_Q)
    audit.reads("qk_0#0", 0, "load_Q#0:out0")
    original = copies[INITIAL_Q]
    donor_span = audit.byte_span(original)
    check(original["occupied_bytes"] == 16384, "full Q donor must occupy 16 KiB")
    stored = {event["id"] + ":out0" for event in events.values() if event["kind"] == "store_r2s"}
    check(stored == {name for name in moved_in if name.startswith("store_")}, "unexpected checkpoint path")

    certificate = {
        "contract": contract,
        "donor_span_bytes": donor_span,
        "original_q_shared_source_steps": [original["start"], original["end"]],
        "recipients": [],
        "scope": "Address reservation and source-order dependencies; readiness on the GPU is what the emitted waits enforce",
    }
    if arm == "retain":
        q_registers = events["qk_1#0"]["inputs"][0]
        if q_registers != "load_Q#0:out0":  # Q was read from the one shared copy a second time
            audit.reads("qk_1#0", 0, "load_Q#1:out0")
            audit.reads("load_Q#1", 0, INITIAL_Q)
        certificate["qk1_q_register_source"] = q_registers
        return certificate

    # -- Q is copied again, elsewhere, for the second score product
    audit.reads("load_Q#1", 0, RESTORED_Q)
    audit.reads("qk_1#0", 0, "load_Q#1:out0")
    second_q = copies[RESTORED_Q]
    second_span = audit.byte_span(second_q)
    check(second_q["occupied_bytes"] == original["occupied_bytes"] and _disjoint(second_span, donor_span),
          "restore Q must use a disjoint address range")
    check(events["qk_0#0"]["end"] <= second_q["start"], "restore must follow the original QK")
    check(copies["load_Q#0:out0"]["end"] == events["qk_0#0"]["end"], "original Q RF held beyond first QK")
    certificate.update(restore_span_bytes=second_span, restore_issue_source_step=second_q["start"])

    # -- the checkpointed probabilities (and, for `multi`, the V stripe) and their ordering
    audit.checkpoint_path(0, 2)
    audit.in_source_order("pv_0_0#0", "qk_1#0", "load_P0#0")
    if arm == "multi":
        audit.reads("load_V0_1#0", 0, V)
        audit.reads("pv_0_1#0", 1, "load_V0_1#0:out0")
        audit.in_source_order("copy_Q#1", "load_V0_1#0")
    if arm == "relocated_two_p":
        audit.checkpoint_path(1, 3)
        audit.in_source_order("store_P1#0", "load_P0#0")

    # -- the recipients live in the vacated range, after the donor, with a consumer still to come
    tenants = [copies[name] for name in moved_in]
    for tenant in tenants:
        tenant_span = audit.byte_span(tenant)
        inside = donor_span[0] <= tenant_span[0] and tenant_span[1] <= donor_span[1]
        check(inside and tenant_span[1] - tenant_span[0] == audit.slab,
              f"recipient {tenant['id']} must occupy one slab in the vacated donor")
        check(original["end"] <= tenant["start"] and tenant["available"] < tenant["end"],
              f"recipient {tenant['id']} has invalid donor reuse or no later consumer")
        certificate["recipients"].append({"copy": tenant["id"], "span_bytes": tenant_span,
                                          "source_steps": [tenant["start"], tenant["end"]],
                                          "producer_end": tenant["available"]})

    # -- between "recipient produced" and "Q copied again" nobody else may sit in the donor's range
    before_restore = tenants[:1] if arm == "relocated_two_p" else tenants
    window = [max(tenant["available"] for tenant in before_restore), second_q["start"]]
    check(window[0] < window[1] <= min(tenant["end"] for tenant in before_restore), "no pre-restore recipient window")
    certificate["pre_restore_reservation_source_steps"] = window
    declared = {INITIAL_Q, RESTORED_Q, *moved_in}
    for other in copies.values():
        if other["tier"] == "smem" and other["id"] not in declared:
            outside_window = other["end"] <= window[0] or window[1] <= other["start"]
            check(outside_window or _disjoint(audit.byte_span(other), donor_span),
                  f"undeclared occupant {other['id']} in the pre-restore window")

    # -- all recipients are resident together for a while, in different slabs
    together = [max(tenant["available"] for tenant in tenants), min(tenant["end"] for tenant in tenants)]
    check(together[0] < together[1], "no common recipient reservation window")
    if len(tenants) == 2:
        check(_disjoint(audit.byte_span(tenants[0]), audit.byte_span(tenants[1])),
              "simultaneous recipients overlap in address")
    if arm == "relocated_two_p":
        check(second_q["available"] <= together[0], "P1 is not available before Q is restored elsewhere")
    certificate["joint_reservation_source_steps"] = together
    return certificate


def _run_arm(arm, directory, seconds, emit_sources):
    """Plan, verify and (optionally) emit one arm into ``directory``; returns a one-line report."""
    problem = build_problem(arm)
    result = model.solve(problem, max_time_seconds=seconds, artifact_dir=directory / "solver")
    certificate = verify(problem.provenance[PROVENANCE_KEY], result)
    (directory / "residency_certificate.json").write_text(json.dumps(certificate, indent=2) + "\n")
    if emit_sources:
        from .emit_exchange import emit

        emit(problem, result, directory / "emitted")
    return f"{result['status']}; {result['finish_step']} source steps"


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--out", required=True, type=Path, help="directory to create; one sub-directory per arm")
    parser.add_argument("--arm", action="append", choices=ARMS, help="repeatable; default: all four arms")
    parser.add_argument("--seconds", type=float, default=15, help="search budget per arm (scales a node budget)")
    parser.add_argument("--no-emit", action="store_true", help="plan and verify only")
    arguments = parser.parse_args(argv)
    model.require(0 < arguments.seconds <= 120, "Per-arm search budget must be between zero and 120 seconds")
    chosen = list(arguments.arm or ARMS)
    model.require(len(chosen) == len(set(chosen)), "Each arm may only be generated once")
    arguments.out.mkdir(parents=True, exist_ok=False)
    failed = []
    for arm in chosen:
        directory = arguments.out / arm
        directory.mkdir()
        try:
            report = _run_arm(arm, directory, arguments.seconds, not arguments.no_emit)
        except (ValueError, RuntimeError) as error:
            (directory / "failure.txt").write_text(f"{error}\n")
            failed.append(arm)
            report = str(error)
        print(f"{arm}: {report}", flush=True)
    if failed:
        raise SystemExit("Unsuccessful arms: " + ", ".join(failed))


if __name__ == "__main__":
    main()

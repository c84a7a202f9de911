"""Pin the exchange planner's verifier and lowering oracle to the reference's own.

Run where the reference tree is available:

    python tests/golden/make_exchange_golden.py /path/to/TileCadence

For every arm it solves the plan with this repository's planner, then asks the REFERENCE's
``exchange.verify`` (``tilecadence/exchange.py:165-289``) for the residency certificate and the
reference's ``model.lowering_trace`` (``tilecadence/model.py:406-494``) for the ready/mask trace of that
plan, and stores plan, certificate and trace in ``exchange_golden.json``. It also stores the trace the
reference computes for the hand-built nine-event sequence of its own unit test
(``tests/test_exchange.py:17-59``).

The plan is then handed to the REFERENCE's full ``model.replay`` (``tilecadence/model.py:1205-1355``)
together with the reference's own problem for that arm (``exchange.build_problem``, the reference
geometry), and what ``replay`` returns is stored as ``reference_replay``. ``replay`` compares a result's
declarations with its problem's, so ``reference_form`` first swaps in the reference problem's texts
(provenance, cost records, value layout descriptions) and the reference's complete source-feature
record, which is a superset of what this planner reports. Everything the planner decides, that is the
events with their order and port bindings, the copies with lifetimes and byte offsets, the objective, its
features and bound, goes through unchanged, and the script stops if the reference recomputes any of
them differently.
"""
import importlib.util
import json
from pathlib import Path
import sys
import types

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from tilecadence_b200 import exchange, model  # noqa: E402


def load_reference(root):
    root = Path(root) / "tilecadence"
    package = types.ModuleType("tilecadence_reference")
    package.__path__ = [str(root)]
    sys.modules["tilecadence_reference"] = package
    modules = {}
    for name in ("model", "exchange"):
        spec = importlib.util.spec_from_file_location(f"tilecadence_reference.{name}", root / f"{name}.py")
        module = importlib.util.module_from_spec(spec)
        sys.modules[spec.name] = module
        spec.loader.exec_module(module)
        modules[name] = module
    return modules["model"], modules["exchange"]


def frontier_case():
    """The hand-built sequence of the reference's CheckpointFrontier test, as plain data."""
    shared = [("issue_q", "q", None, 0, 16384), ("issue_v", "v", 0, 16384, 4096), ("store_p", "p", None, 0, 4096),
              ("issue_k", "k", None, 0, 8192)]
    copies = [dict(id=name, producer=name, role=role, stripe=stripe, tier="smem", offset_bytes=offset,
                   occupied_bytes=width) for name, role, stripe, offset, width in shared]
    sequence = [("issue_q", "copy_g2s", [], ["issue_q"]), ("read_q", "load_s2r", ["issue_q"], ["q_rf"]),
                ("issue_v", "copy_g2s", [], ["issue_v"]), ("store_p", "store_r2s", [], ["store_p"]),
                ("read_p", "load_s2r", ["store_p"], ["p_rf"]), ("read_v", "load_s2r", ["issue_v"], ["v_rf"]),
                ("read_p_again", "load_s2r", ["store_p"], ["p_rf"]), ("read_v_again", "load_s2r", ["issue_v"], ["v_rf"]),
                ("issue_k", "copy_g2s", [], ["issue_k"])]
    copies.extend({"id": name, "tier": "reg"} for name in ("q_rf", "p_rf", "v_rf"))
    events = [dict(id=name, kind=kind, start=step, end=step + 1, inputs=inputs, outputs=outputs)
              for step, (name, kind, inputs, outputs) in enumerate(sequence)]
    provenance = {"residency_exchange_v78": {}, "execution_mode": "source_order",
                  "backend_spec": {"close_workspace_smem_bytes": 8192}}
    return provenance, {"copies": copies, "events": events}


def reference_form(ref_model, ref_problem, result):
    """``result`` with the reference problem's declarative texts; see the module docstring."""
    from dataclasses import asdict

    converted = json.loads(json.dumps(result))
    converted["actions"] = converted["events"]
    values = {v.name: v for v in ref_problem.values}
    actions = {a["id"]: a for a in ref_problem.actions}
    for copy in converted["copies"]:
        if copy["workspace"]:
            copy["layout"] = ref_model._workspace_value(actions[copy["producer"]]).layout
        else:
            copy["layout"] = values[copy["value"]].layout
    converted["profiles"] = {key: asdict(cost) for key, cost in ref_problem.profiles.items()}
    converted["provenance"] = dict(ref_problem.provenance)
    converted["source_features"] = ref_model.source_feature_values(ref_problem, converted)
    ordered = sorted(converted["events"], key=lambda e: (e["start"], e["id"]))
    # decisions and their prices must come out of the reference's own arithmetic unchanged
    assert converted["objective"] == ref_model.evaluate_objective(ref_problem, ordered, converted)
    assert converted["objective_features"] == ref_model.objective_features(ref_problem, ordered, converted)
    assert converted["lowering_trace"] == ref_model.lowering_trace(ref_problem, converted)
    assert converted["objective_model"]["spec"] == ref_problem.objective_spec
    assert all(converted["source_features"][key] == value for key, value in result["source_features"].items()
               if key in converted["source_features"])
    return converted


def main():
    if len(sys.argv) != 2:
        sys.exit(f"usage: python {sys.argv[0]} /path/to/TileCadence")
    ref_model, ref_exchange = load_reference(sys.argv[1])
    golden = {"arms": {}}
    for arm in exchange.ARMS:
        problem = exchange.build_problem(arm)
        result = model.solve(problem, max_time_seconds=2)
        plan = {"events": result["events"], "copies": result["copies"], "status": result["status"]}
        replayed = ref_model.replay(ref_exchange.build_problem(arm), reference_form(ref_model, ref_exchange.build_problem(arm), result))
        replayed.pop("note")
        golden["arms"][arm] = {
            "plan": plan,
            "reference_certificate": ref_exchange.verify(ref_exchange.build_contract(arm), result),
            "reference_trace": ref_model.lowering_trace(problem, result),
            "reference_replay": replayed,
        }
    provenance, record = frontier_case()
    golden["frontier"] = {"provenance": provenance, "record": record,
                          "reference_trace": ref_model.lowering_trace(types.SimpleNamespace(provenance=provenance), record)}
    target = Path(__file__).with_name("exchange_golden.json")
    target.write_text(json.dumps(golden, separators=(",", ":")) + "\n")
    print(target, target.stat().st_size, "bytes")


if __name__ == "__main__":
    main()

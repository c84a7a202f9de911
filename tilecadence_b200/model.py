"""Two-KV-tile attention action graph, source-order planner, lowering oracle and replay.

Counterpart of ``tilecadence/model.py`` for the residency-exchange study (the only caller the
reference ships is ``tilecadence/exchange.py``): one CTA computes complete attention for 64 queries
over two key tiles of 32 (D = 128, two 64-wide output stripes) as a straight line of *actions* —
global-to-shared copies, shared-to-register loads, register-to-shared checkpoints and the math
steps — and the planner chooses their source order, the register/shared copy every operand port
reads and the 4 KiB slab every shared copy occupies.

What is kept from the reference, because other modules and the tests speak this vocabulary:
action and copy identities (``qk_0#0``, ``stats_1#0:out3``, ``copy_Q#1:out0`` ...; graph built at
``model.py:201-354``), the result dictionary (``events`` with ``profile_key`` / ``profile_cost``,
``copies`` including the initial global-memory copies, ``output_states``, ``lowering_trace``,
``source_features``, ``objective_features``, ``profiles``, ``best_bound``, ``lexicographic_objective``,
``model_sha256``; ``model.py:1131-1197``) in the form the reference's own ``replay`` accepts, the ordinal lowering oracle
(``lowering_trace``, ``model.py:406-494``) and an independent ``replay`` (``model.py:1205-1355``)
that raises ``ValueError`` on any inconsistency.

What is new: there is no CP-SAT. ``solve`` binds every operand port from the declarative residency
contract, then runs a depth-first branch-and-bound over source orders with slab allocation on the
fly, minimising the reference's objective (128 per selected action + register KiB-steps). The
lowering oracle is stated for Blackwell: every ``copy_g2s`` is a TMA tile copy that arms its own
transaction mbarrier; the "ready cutoff" is the newest copy whose barrier the whole CTA has
observed, and an operand load newer than the cutoff first observes every barrier armed so far and
joins a CTA barrier (the arithmetic is the reference's wait-all-groups rule, so its certificates
carry over unchanged).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field
import hashlib
import json
import math
from pathlib import Path
import time
from typing import Any, Mapping

SLAB_BYTES = 4096
OUTPUT_STRIPE_BYTES = 16384
MODEL_REVISION = "b200-two-tile-source-order-dfs-v1"
SHAPE = {"M": 64, "N": 32, "D": 128, "Dv_stripe": 64, "warps": 4, "kv_tiles": 2}
ACTION_KINDS = {"copy_g2s", "load_s2r", "store_r2s", "qk", "stats_first", "stats_next", "pv_first", "pv_next",
                "rescale_o", "normalize_store", "store_lse"}
# Tensor-core / exponential instruction sites of one action per warp; the oracle accumulates them
# between the last copy issue and the next wait to show how much math overlaps a copy in flight.
MATH_SITE_WEIGHTS = {"qk": (32, 0), "pv_first": (16, 0), "pv_next": (16, 0), "stats_first": (0, 16),
                     "stats_next": (0, 18)}
REGISTER_REPLICATION = {"q": 1, "k": 4, "v": 4, "s": 1, "p": 1, "m": 4, "l": 4, "alpha": 4}
MAX_OUTSTANDING_COPIES = 8
NODES_PER_SECOND = 20000


def require(condition, message):
    if not condition:
        raise ValueError(message)


def integer(x, minimum=0):
    return isinstance(x, int) and not isinstance(x, bool) and x >= minimum


@dataclass(frozen=True)
class Value:
    name: str
    role: str
    tile: int | None
    stripe: int | None
    logical_bytes: int
    register_bytes: int
    layout: str


@dataclass(frozen=True)
class Problem:
    values: tuple[Value, ...]
    actions: tuple[Mapping[str, Any], ...]
    arena_slabs: int
    register_budget_bytes: int
    precedence_edges: tuple[tuple[str, str], ...]
    state_chains: tuple[tuple[str, ...], ...]
    kv_order: tuple[int, ...]
    objective_spec: Mapping[str, Any]
    provenance: Mapping[str, Any]
    plan: Mapping[str, Any] = field(default_factory=dict)  # declarative residency constraints
    profiles: Mapping[str, Any] = field(default_factory=dict)  # profile_key -> declared cost record


def _occupied(value, tier):
    return value.register_bytes if tier == "reg" else math.ceil(value.logical_bytes / SLAB_BYTES) * SLAB_BYTES


def build_problem(*, arena_slabs=8, register_budget_bytes=98304, allow_probability_spill=True, objective_spec=None,
                  close_workspace_smem_bytes=8192, provenance=None, plan=None, kv_order=(0, 1)):
    """Value and action vocabulary of the two-tile kernel (``model.py:201-354`` restricted to what the
    exchange study uses: one QK per tile, no score spill, no P recomputation, split-V stripes)."""
    require(arena_slabs in (4, 8) and integer(register_budget_bytes, 1), "Bounded 4 KiB-unit arena and positive RF budget required")
    require(tuple(kv_order) == (0, 1), "Key tiles are consumed in order 0, 1")
    require(close_workspace_smem_bytes == 8192, "The coalesced close needs one declared 8 KiB scratch span")
    require(isinstance(objective_spec, dict) and objective_spec.get("terms"), "Supply an affine objective")

    def value(name, role, tile, stripe, logical, layout):
        return Value(name, role, tile, stripe, logical, logical * REGISTER_REPLICATION[role], layout)

    values = [value("Q", "q", None, None, 16384, "M64xD128 A operand, two 128-byte-swizzled halves")]
    for j in (0, 1):
        values += [value(f"K{j}", "k", j, None, 8192, "N32xD128 B operand, two swizzled halves"),
                   value(f"S{j}", "s", j, None, 8192, "M64xN32 FP32 accumulator"),
                   value(f"P{j}", "p", j, None, 4096, "M64xN32 input-dtype A operand"),
                   value(f"m{j}", "m", j, None, 256, "FP32 running row maximum"),
                   value(f"l{j}", "l", j, None, 256, "FP32 full row sum")]
        values += [value(f"V{j}_{s}", "v", j, s, 4096, "N32xDv64 B operand, one swizzled box") for s in (0, 1)]
    values.append(value("alpha1", "alpha", 1, None, 256, "FP32 online rescale factor"))
    actions = []
    roles = {v.name: v.role for v in values}

    def profile_of(kind, inputs, outputs):
        """Name of the action's cost record (the reference's primitive vocabulary, ``model.py:201-354``)."""
        moved = roles[(outputs or inputs)[0][0]] if kind in ("copy_g2s", "load_s2r", "store_r2s") else None
        wide = "64" if moved == "v" else ""
        return {"copy_g2s": f"copy_{moved}{wide}", "load_s2r": f"load_{moved}{wide}", "store_r2s": f"store_{moved}",
                "qk": "qk", "stats_first": "stats_emit_p_first", "stats_next": "stats_emit_p_next",
                "pv_first": "pv64_first", "pv_next": "pv64_next", "rescale_o": "rescale_o64",
                "normalize_store": "normalize_store64", "store_lse": "store_lse"}[kind]

    def add(name, kind, inputs, outputs, maximum=1, mandatory=False, tile=None, stripe=None, first=False):
        for instance in range(maximum):
            actions.append({"id": f"{name}#{instance}", "name": name, "instance": instance, "kind": kind,
                            "input_refs": [list(x) for x in inputs], "output_refs": [list(x) for x in outputs],
                            "profile_key": profile_of(kind, inputs, outputs), "profile_cost": 0,
                            "duration": 1, "mandatory": mandatory, "tile": tile, "stripe": stripe, "first": first,
                            "value": outputs[0][0] if len(outputs) == 1 else None, "workspace_reg_bytes": 0,
                            "workspace_smem_bytes": close_workspace_smem_bytes if kind == "normalize_store" else 0})

    for v in values:
        if v.role in ("q", "k", "v"):
            copies = 4 if v.role == "q" else 2
            add("copy_" + v.name, "copy_g2s", ((v.name, "gmem"),), ((v.name, "smem"),), copies, tile=v.tile, stripe=v.stripe)
            add("load_" + v.name, "load_s2r", ((v.name, "smem"),), ((v.name, "reg"),), copies, tile=v.tile, stripe=v.stripe)
        elif v.role == "p" and allow_probability_spill:
            add("store_" + v.name, "store_r2s", ((v.name, "reg"),), ((v.name, "smem"),), 1, tile=v.tile)
            add("load_" + v.name, "load_s2r", ((v.name, "smem"),), ((v.name, "reg"),), 2, tile=v.tile)
    for step, j in enumerate(kv_order):
        add(f"qk_{j}", "qk", (("Q", "reg"), (f"K{j}", "reg")), ((f"S{j}", "reg"),), tile=j)
        ins = ((f"S{j}", "reg"),) if step == 0 else ((f"S{j}", "reg"), ("m0", "reg"), ("l0", "reg"))
        outs = ((f"m{j}", "reg"), (f"l{j}", "reg")) + (() if step == 0 else (("alpha1", "reg"),)) + ((f"P{j}", "reg"),)
        add(f"stats_{j}", "stats_first" if step == 0 else "stats_next", ins, outs, mandatory=True, tile=j, first=step == 0)
    chains = []
    for s in (0, 1):
        add(f"pv_0_{s}", "pv_first", (("P0", "reg"), (f"V0_{s}", "reg")), (), mandatory=True, tile=0, stripe=s, first=True)
        add(f"rescale_1_{s}", "rescale_o", (("alpha1", "reg"),), (), mandatory=True, tile=1, stripe=s)
        add(f"pv_1_{s}", "pv_next", (("P1", "reg"), (f"V1_{s}", "reg")), (), mandatory=True, tile=1, stripe=s)
        add(f"close_{s}", "normalize_store", (("l1", "reg"),), (), mandatory=True, stripe=s)
        chains.append((f"pv_0_{s}#0", f"rescale_1_{s}#0", f"pv_1_{s}#0", f"close_{s}#0"))
    add("store_lse", "store_lse", (("m1", "reg"), ("l1", "reg")), (), mandatory=True)
    edges = [("stats_0#0", "stats_1#0")]
    for chain in chains:
        edges.extend(zip(chain, chain[1:]))
    return Problem(tuple(values), tuple(actions), arena_slabs, register_budget_bytes, tuple(edges), tuple(chains),
                   tuple(kv_order), json.loads(json.dumps(objective_spec)), {
                       **dict(provenance or {}), "shape": dict(SHAPE), "model_revision": MODEL_REVISION,
                       "ordering_unit": "source_steps", "execution_mode": "source_order",
                       "objective_unit": objective_spec.get("unit", "cost_ticks"),
                       "backend_spec": {"name": "sm100a-tma-mbarrier-mma-primitives", "shared_slab_bytes": SLAB_BYTES,
                                        "register_replication_by_role": dict(REGISTER_REPLICATION),
                                        "row_sum_representation": "full_sum_quad_replicated",
                                        "copy_semantics": "async_issue_ready_mask_wait",
                                        "copy_engine": "TMA tile copy, one transaction mbarrier per copy",
                                        "close_workspace_smem_bytes": close_workspace_smem_bytes},
                       "O_state_bytes_per_stripe": OUTPUT_STRIPE_BYTES,
                       "limitation": "Source dependency and address intervals only; completion on the GPU is what the emitted waits enforce"},
                   dict(plan or {}),
                   # Every primitive is unpriced: the objective is the affine whole-plan proxy, not a sum of latencies.
                   {key: {"duration": 0, "kind": "derived", "unit": objective_spec.get("unit", "cost_ticks"),
                          "provenance": {"scope": "Unpriced primitive; the affine whole-plan objective ignores it",
                                         "not_a_primitive_latency": True}}
                    for key in sorted({a["profile_key"] for a in actions})})


def problem_to_dict(p):
    return json.loads(json.dumps(asdict(p)))


def problem_from_dict(d):
    return Problem(tuple(Value(**v) for v in d["values"]), tuple(d["actions"]), d["arena_slabs"],
                   d["register_budget_bytes"], tuple(tuple(e) for e in d["precedence_edges"]),
                   tuple(tuple(c) for c in d["state_chains"]), tuple(d["kv_order"]), d["objective_spec"],
                   d["provenance"], d.get("plan", {}), d.get("profiles", {}))


def validate_problem(p):
    """Structural validation of ports, sizes and edges (``model.py:577-684``)."""
    values = {v.name: v for v in p.values}
    require(len(values) == len(p.values), "Duplicate value names")
    for v in p.values:
        require(v.role in REGISTER_REPLICATION and integer(v.logical_bytes, 1)
                and v.register_bytes == v.logical_bytes * REGISTER_REPLICATION[v.role], f"Bad value geometry for {v.name}")
    ids = [a["id"] for a in p.actions]
    require(len(ids) == len(set(ids)), "Duplicate action identities")
    for a in p.actions:
        require(a["kind"] in ACTION_KINDS and a["duration"] == 1, f"Bad action {a['id']}")
        require(not p.profiles or a.get("profile_key") in p.profiles, f"Action {a['id']} names an undeclared cost record")
        for name, tier in [*a["input_refs"], *a["output_refs"]]:
            require(name in values and tier in ("gmem", "smem", "reg"), f"Unknown port value in {a['id']}")
        if a["kind"] == "copy_g2s":
            require(a["input_refs"][0][1] == "gmem" and a["output_refs"][0][1] == "smem", "copy_g2s moves global to shared")
        if a["kind"] == "load_s2r":
            require(a["input_refs"][0][1] == "smem" and a["output_refs"][0][1] == "reg", "load_s2r moves shared to registers")
        if a["kind"] == "store_r2s":
            require(a["input_refs"][0][1] == "reg" and a["output_refs"][0][1] == "smem", "store_r2s moves registers to shared")
    known = set(ids)
    require(all(a in known and b in known and a != b for a, b in p.precedence_edges), "Unknown/self precedence edge")
    require(all(set(chain) <= known for chain in p.state_chains), "Unknown action in an output-state chain")
    require(p.provenance.get("shape") == SHAPE, "Fixed M64/N32/D128/two-stripe geometry")
    return True


def _slab_mask(copy):
    require(copy["offset_bytes"] % SLAB_BYTES == 0 and copy["occupied_bytes"] % SLAB_BYTES == 0, "Invalid physical slab span")
    return ((1 << (copy["occupied_bytes"] // SLAB_BYTES)) - 1) << (copy["offset_bytes"] // SLAB_BYTES)


def lowering_trace(p, r):
    """CPU oracle of the emitted synchronisation: copy readiness cutoff and pending shared reads.

    Every ``copy_g2s`` arms a fresh mbarrier (``issued_groups`` counts them). An operand load whose
    producing copy ended after the ready cutoff must wait: the CTA observes every barrier armed so
    far and meets at a CTA barrier, which moves the cutoff to this step, marks all copies ready and
    retires every earlier distributed shared read. A shared write (copy, checkpoint store, close
    scratch) that overlaps a slab still being read forces a CTA release first. Checkpoint stores and
    the close end with a CTA barrier of their own, which retires reads but says nothing about copies
    in flight. Same arithmetic as ``model.py:406-494``; ordinal, not elapsed time.
    """
    require(p.provenance["execution_mode"] == "source_order"
            and p.provenance["backend_spec"]["close_workspace_smem_bytes"] == 8192,
            "Ready-aware lowering requires source order and the 8 KiB close scratch")
    require(all(e["kind"] in ACTION_KINDS for e in r["events"]), "Unsupported action kind in the lowering oracle")
    copies = {c["id"]: c for c in r["copies"]}
    events = {e["id"]: e for e in r["events"]}
    pending: dict[str, dict] = {}
    trace = []
    cutoff = issued = ready = hmma_gap = ex2_gap = 0

    def read_mask():
        mask = 0
        for copy in pending.values():
            mask |= _slab_mask(copy)
        return mask

    for e in sorted(r["events"], key=lambda e: e["start"]):
        row = {"id": e["id"], "kind": e["kind"], "frontier_before": sorted(pending), "read_mask_before": read_mask(),
               "ready_cutoff_before": cutoff, "issued_groups_before": issued, "ready_groups_before": ready,
               "last_commit_hmma_before": hmma_gap, "last_commit_ex2_before": ex2_gap}
        writes = []
        if e["kind"] in ("copy_g2s", "store_r2s"):
            writes = [copies[x] for x in e["outputs"] if copies[x]["tier"] == "smem"]
        elif e["kind"] == "normalize_store":
            require(len(e.get("workspace_copies", [])) == 1, "The close needs exactly one scratch span")
            writes = [copies[e["workspace_copies"][0]]]
        require(len(writes) <= 1, "At most one shared write per action")
        hazards = [[w["id"], identity] for w in writes for identity, c in pending.items() if _slab_mask(w) & _slab_mask(c)]
        if hazards:
            pending.clear()
        wait, producer_end = False, 0
        if e["kind"] == "copy_g2s":
            issued += 1
        elif e["kind"] == "load_s2r":
            require(len(e["inputs"]) == 1, "A shared load has one source")
            source = copies[e["inputs"][0]]
            producer = events[source["producer"]]
            require(producer["end"] <= e["start"], "A shared load must follow its producer")
            if source["role"] in ("q", "k", "v"):
                require(producer["kind"] == "copy_g2s", "An operand load reads an input copy")
                producer_end = producer["end"]
                wait = producer_end > cutoff
                if wait:
                    pending.clear()
                    cutoff, ready = e["end"], issued
            else:
                require(source["role"] == "p" and producer["kind"] == "store_r2s", "A checkpoint load reads a checkpoint store")
            pending[source["id"]] = source
        elif e["kind"] == "store_r2s":
            pending.clear()
        elif e["kind"] == "normalize_store":
            pending.clear()
            pending[writes[0]["id"]] = writes[0]
        require(0 <= ready <= issued and issued - ready <= MAX_OUTSTANDING_COPIES, "Too many copies in flight")
        wait_hmma, wait_ex2 = (hmma_gap, ex2_gap) if wait else (0, 0)
        if e["kind"] == "copy_g2s" or wait:
            hmma_gap = ex2_gap = 0
        else:
            hmma, ex2 = MATH_SITE_WEIGHTS.get(e["kind"], (0, 0))
            hmma_gap, ex2_gap = hmma_gap + hmma, ex2_gap + ex2
        row.update({"write_role": writes[0]["role"] if writes else None, "frontier_after": sorted(pending),
                    "read_mask_after": read_mask(), "ready_cutoff_after": cutoff, "producer_end": producer_end,
                    "wait_before_load": wait, "acquire_before_load": wait, "issued_groups_after": issued,
                    "ready_groups_after": ready, "last_commit_hmma_after": hmma_gap, "last_commit_ex2_after": ex2_gap,
                    "last_commit_wait_hmma_sites": wait_hmma, "last_commit_wait_ex2_sites": wait_ex2,
                    "release_before_write": bool(hazards), "shared_read_write_hazards": hazards})
        trace.append(row)
    return trace


def _kib(size):
    require(size % 1024 == 0, "KiB-step features need whole-KiB payloads")
    return size // 1024


def source_feature_values(p, r):
    """Order- and lifetime-derived features of a plan (the subset of ``model.py:497-562`` the
    exchange objective and reports use)."""
    regs = [c for c in r["copies"] if c["tier"] == "reg"]
    trace = lowering_trace(p, r)
    steps = range(r["finish_step"])
    return {
        "rf_kib_steps": sum(_kib(c["occupied_bytes"]) * (c["end"] - c["start"]) for c in regs)
        + sum(_kib(s["bytes"]) * (s["end"] - s["start"]) for s in r["output_states"]),
        "o_kib_steps": sum(_kib(s["bytes"]) * (s["end"] - s["start"]) for s in r["output_states"]),
        "rf_peak_kib": max(sum(_kib(c["occupied_bytes"]) for c in regs if c["start"] <= t < c["end"])
                           + sum(_kib(s["bytes"]) for s in r["output_states"] if s["start"] <= t < s["end"])
                           for t in steps),
        "consumer_wait_count": sum(row["wait_before_load"] for row in trace),
        # releases in front of input copies and the close's scratch, as the reference counts them
        # (model.py:507-510); a checkpoint store's release is part of the checkpoint's own cost
        "release_barrier_count": sum(row["release_before_write"] and row["kind"] in ("copy_g2s", "normalize_store")
                                     for row in trace),
        "last_commit_wait_hmma_sites": sum(row["last_commit_wait_hmma_sites"] for row in trace),
        "last_commit_wait_ex2_sites": sum(row["last_commit_wait_ex2_sites"] for row in trace),
        "source_actions": len(r["events"]),
    }


def _term_source(term):
    """Which plan feature an objective term prices. Two spellings are read: this package's
    ``{"feature": "rf_kib_steps"}`` and the reference's (``exchange.py:47-55``), where ``feature`` is a label, a
    ``source`` record names an order-derived feature and an empty ``match`` counts every selected action."""
    if "source" in term:
        require(set(term["source"]) == {"kind"}, "Only plain source features are priced")
        return term["source"]["kind"]
    if "match" in term:
        require(term["match"] == {}, "Only the all-actions match is priced")
        return "source_actions"
    return term["feature"]


def objective_features(p, r):
    """Value of every objective term, keyed by the term's label (``model.py:138-147``)."""
    features = source_feature_values(p, r)
    for term in p.objective_spec["terms"]:
        require(_term_source(term) in features, f"Unknown objective feature {term['feature']}")
    return {term["feature"]: features[_term_source(term)] for term in p.objective_spec["terms"]}


def evaluate_objective(p, r):
    values = objective_features(p, r)
    return p.objective_spec.get("constant", 0) + sum(term["coefficient"] * values[term["feature"]]
                                                     for term in p.objective_spec["terms"])


# --------------------------------------------------------------------------------------- planner
def _bound_graph(p, overrides):
    """Select the actions a plan needs and bind every input port to a concrete copy.

    Default binding: a port reads output #k of instance 0 of the action that produces that
    (value, tier); ``p.plan['bindings']`` and ``overrides`` ({"consumer:port": copy}) replace it.
    The selection is the closure of the mandatory actions and ``p.plan['selected']`` under "the
    producer of every bound copy is selected".
    """
    actions = {a["id"]: a for a in p.actions}
    values = {v.name: v for v in p.values}
    producers = {}
    for prefer_math in (True, False):  # a register value comes from the math that defines it unless the plan says otherwise
        for a in p.actions:
            if a["instance"] == 0 and (a["kind"] != "load_s2r") == prefer_math:
                for index, (name, tier) in enumerate(a["output_refs"]):
                    producers.setdefault((name, tier), f"{a['id']}:out{index}")
    explicit = {**{f"{c}:{port}": copy for c, ports in p.plan.get("bindings", {}).items() for port, copy in ports.items()},
                **overrides}
    forbidden = set(p.plan.get("forbidden", ()))
    selected, frontier, inputs = {}, [a["id"] for a in p.actions if a["mandatory"]] + list(p.plan.get("selected", ())), {}
    ports = {}  # every input port in declaration order, global-memory ports included (what the events record)
    while frontier:
        identity = frontier.pop()
        if identity in selected:
            continue
        require(identity in actions and identity not in forbidden, f"Plan needs unavailable action {identity}")
        action = actions[identity]
        selected[identity] = action
        bound, ports[identity] = [], []
        for port, (name, tier) in enumerate(action["input_refs"]):
            if tier == "gmem":
                ports[identity].append("gmem:" + name)
                continue
            copy = explicit.get(f"{identity}:{port}", producers.get((name, tier)))
            require(copy is not None, f"No producer for port {port} of {identity}")
            producer, _, out = copy.partition(":out")
            require(producer in actions and list(actions[producer]["output_refs"][int(out)]) == [name, tier],
                    f"{copy} does not carry ({name}, {tier}) for {identity}")
            bound.append(copy)
            ports[identity].append(copy)
            frontier.append(producer)
        inputs[identity] = bound
    copies = {}
    for identity, action in selected.items():
        for index, (name, tier) in enumerate(action["output_refs"]):
            v = values[name]
            copies[f"{identity}:out{index}"] = dict(
                id=f"{identity}:out{index}", value=name, role=v.role, tile=v.tile, stripe=v.stripe, tier=tier,
                logical_bytes=v.logical_bytes, nbytes=v.logical_bytes, occupied_bytes=_occupied(v, tier),
                layout=v.layout, producer=identity, workspace=False)
        if action["workspace_smem_bytes"]:
            copies[_workspace_id(identity)] = dict(
                id=_workspace_id(identity), value="__workspace:" + identity, role="workspace", tile=None,
                stripe=action["stripe"], tier="smem", logical_bytes=action["workspace_smem_bytes"],
                nbytes=action["workspace_smem_bytes"], occupied_bytes=action["workspace_smem_bytes"],
                layout="close scratch, internal to the action", producer=identity, workspace=True)
    consumers = {identity: [] for identity in copies}
    for identity, bound in inputs.items():
        for copy in bound:
            require(copy in copies, f"{identity} reads {copy}, which no selected action produces")
            consumers[copy].append(identity)
    return selected, inputs, copies, consumers, ports


def _workspace_id(action_id):
    return "workspace:" + action_id


class _Search:
    """Depth-first branch-and-bound over source orders with slab allocation on the fly."""

    KIND_RANK = {"store_lse": 0, "normalize_store": 1, "pv_next": 2, "pv_first": 2, "rescale_o": 3, "stats_next": 4,
                 "stats_first": 4, "qk": 5, "store_r2s": 6, "load_s2r": 7, "copy_g2s": 8}

    def __init__(self, p, graph, node_budget):
        self.p, self.node_budget = p, node_budget
        self.selected, self.inputs, self.copies, self.consumers, _ = graph
        self.order = sorted(self.selected)
        self.bit = {identity: 1 << i for i, identity in enumerate(self.order)}
        plan = p.plan
        self.donor, self.restore = plan.get("donor"), plan.get("restore")
        self.recipients = tuple(plan.get("recipients", ()))
        self.window_open = tuple(plan.get("window_open", ()))
        self.slabs = p.arena_slabs
        preds = {identity: set() for identity in self.selected}
        for identity, bound in self.inputs.items():
            preds[identity].update(copy.partition(":out")[0] for copy in bound)
        self.gaps = {identity: [] for identity in self.selected}  # b -> [(a, idle steps required between them)]
        for a, b, *gap in [*p.precedence_edges, *plan.get("before", ())]:
            if a in self.selected and b in self.selected:
                preds[b].add(a)
                if gap and gap[0]:
                    self.gaps[b].append((a, gap[0]))
        # A recipient may only be written after the donor copy has been read for the last time.
        if self.donor in self.copies:
            for recipient in self.recipients:
                preds[recipient.partition(":out")[0]].update(self.consumers[self.donor])
        self.pred_mask = {identity: sum(self.bit[x] for x in ps) for identity, ps in preds.items()}
        self.chain_of = {}
        for stripe, chain in enumerate(p.state_chains):
            self.chain_of[chain[0]] = ("open", stripe)
            self.chain_of[chain[-1]] = ("close", stripe)
        self.best_cost, self.best_plan, self.nodes, self.complete = None, None, 0, True
        self.memo = {}
        self.fixed_cost = 0
        for term in p.objective_spec["terms"]:
            if _term_source(term) == "source_actions":
                self.fixed_cost += term["coefficient"] * len(self.selected)
            elif _term_source(term) == "rf_kib_steps":
                self.rf_weight = term["coefficient"]
        self.rf_weight = getattr(self, "rf_weight", 0)

    # ---- address rules ------------------------------------------------------------------
    def _candidates(self, copy_id, slabs_needed, occupied, donor_span, window):
        free = [all((offset + i) not in occupied for i in range(slabs_needed))
                for offset in range(self.slabs - slabs_needed + 1)]
        offsets = [o for o, ok in enumerate(free) if ok]
        if donor_span is not None:
            lo, hi = donor_span
            inside = lambda o: lo <= o and o + slabs_needed <= hi
            apart = lambda o: o + slabs_needed <= lo or hi <= o
            if copy_id in self.recipients:
                offsets = [o for o in offsets if inside(o)]
            elif copy_id == self.restore:
                offsets = [o for o in offsets if apart(o)]
            elif copy_id != self.donor:
                if window:
                    offsets = [o for o in offsets if apart(o)]
                else:  # keep the donor's range free for its future tenants when there is a choice
                    offsets.sort(key=lambda o: (not apart(o), o))
        return offsets[:3]

    def run(self):
        self._dfs(0, 0, {}, {}, {}, set(), {}, None, False, [])
        return self.best_cost, self.best_plan

    def _dfs(self, done, cost, smem, regs, starts, open_states, state_starts, donor_span, window, trail):
        """smem: copy -> (offset_slab, n_slabs); regs: copy -> KiB; trail: [(event, {copy: offset}, freed)]"""
        self.nodes += 1
        if self.nodes > self.node_budget:
            self.complete = False
            return
        if self.best_cost is not None and cost + self.fixed_cost >= self.best_cost:
            return
        if len(trail) == len(self.order):
            self.best_cost, self.best_plan = cost + self.fixed_cost, list(trail)
            return
        key = (done, tuple(sorted((c, o) for c, (o, _) in smem.items())))
        seen = self.memo.get(key)
        if seen is not None and seen <= cost:
            return
        self.memo[key] = cost
        step = len(trail)
        step_of = {identity: index for index, (identity, _, _) in enumerate(trail)}
        ready = [x for x in self.order if not done & self.bit[x] and (self.pred_mask[x] & done) == self.pred_mask[x]
                 and all(step_of[a] + 1 + gap <= step for a, gap in self.gaps[x])]
        ready.sort(key=lambda x: (self.KIND_RANK[self.selected[x]["kind"]], x))
        for identity in ready:
            if self.nodes > self.node_budget:
                return
            action = self.selected[identity]
            new_regs, new_open, new_state_starts = dict(regs), set(open_states), dict(state_starts)
            outputs = [c for c in self.copies if self.copies[c]["producer"] == identity and not self.copies[c]["workspace"]]
            for c in outputs:
                if self.copies[c]["tier"] == "reg":
                    new_regs[c] = _kib(self.copies[c]["occupied_bytes"])
            role = self.chain_of.get(identity)
            if role and role[0] == "open":
                new_open.add(role[1])
                new_state_starts[role[1]] = step
            live_kib = sum(new_regs.values()) + len(new_open) * _kib(OUTPUT_STRIPE_BYTES)
            if live_kib * 1024 > self.p.register_budget_bytes:
                continue
            freed = [c for c in self.inputs[identity] if all(done & self.bit[x] or x == identity for x in self.consumers[c])]
            freed += [c for c in outputs if not self.consumers[c]]
            writes = [c for c in outputs if self.copies[c]["tier"] == "smem"]
            scratch = _workspace_id(identity) if _workspace_id(identity) in self.copies else None
            occupied = {o + i for o, n in smem.values() for i in range(n)}
            placements = [dict()]
            if writes:
                c = writes[0]
                need = self.copies[c]["occupied_bytes"] // SLAB_BYTES
                placements = [{c: o} for o in self._candidates(c, need, occupied, donor_span, window)]
            elif scratch:
                placements = [{scratch: o} for o in self._candidates(scratch, 2, occupied, donor_span, window)][:1]
            for placement in placements:
                new_smem = dict(smem)
                for c, o in placement.items():
                    if c != scratch:
                        new_smem[c] = (o, self.copies[c]["occupied_bytes"] // SLAB_BYTES)
                new_span = donor_span
                if self.donor in placement:
                    new_span = (placement[self.donor], placement[self.donor] + self.copies[self.donor]["occupied_bytes"] // SLAB_BYTES)
                after_regs = {c: k for c, k in new_regs.items() if c not in freed}
                after_smem = {c: v for c, v in new_smem.items() if c not in freed}
                after_open = set(new_open)
                if role and role[0] == "close":
                    after_open.discard(role[1])
                new_window = window
                new_done = done | self.bit[identity]
                if self.restore and identity == self.restore.partition(":out")[0]:
                    new_window = False
                elif self.window_open and not window and new_span is not None and \
                        all(new_done & self.bit[w.partition(":out")[0]] for w in self.window_open) and \
                        not (new_done & self.bit[self.restore.partition(":out")[0]]):
                    lo, hi = new_span
                    exempt = {self.donor, self.restore, *self.recipients}
                    if any(c not in exempt and o < hi and lo < o + n for c, (o, n) in after_smem.items()):
                        continue  # an undeclared tenant would sit in the donor's range when the window opens
                    new_window = True
                trail.append((identity, dict(placement), list(freed)))
                self._dfs(new_done, cost + self.rf_weight * live_kib, after_smem, after_regs, starts, after_open,
                          new_state_starts, new_span, new_window, trail)
                trail.pop()


def _materialise(p, graph, plan_trail, status, complete):
    selected, inputs, copies, consumers, ports = graph
    step_of = {identity: step for step, (identity, _, _) in enumerate(plan_trail)}
    finish = len(plan_trail)
    offsets = {}
    for _, placement, _ in plan_trail:
        offsets.update(placement)
    rows = []
    for identity, c in copies.items():
        producer_step = step_of[c["producer"]]
        row = dict(c, start=producer_step, available=producer_step + 1,
                   end=max([step_of[x] + 1 for x in consumers[identity]] or [producer_step + 1]),
                   offset_bytes=offsets[identity] * SLAB_BYTES if c["tier"] == "smem" else None)
        if c["workspace"]:
            row["end"] = producer_step + 1
        rows.append(row)
    # The kernel's inputs: one global-memory copy per Q/K/V value, present for the whole plan.
    for v in p.values:
        if v.role in ("q", "k", "v"):
            rows.append(dict(id="gmem:" + v.name, value=v.name, role=v.role, tile=v.tile, stripe=v.stripe, tier="gmem",
                             logical_bytes=v.logical_bytes, nbytes=v.logical_bytes, occupied_bytes=v.logical_bytes,
                             layout=v.layout, producer=None, workspace=False, start=0, available=0, end=finish,
                             offset_bytes=None))
    events = []
    for identity, action in selected.items():
        e = {k: action[k] for k in ("id", "name", "kind", "instance", "value", "tile", "stripe", "first", "profile_key",
                                    "duration", "profile_cost", "workspace_reg_bytes", "workspace_smem_bytes")}
        e.update(start=step_of[identity], end=step_of[identity] + 1, inputs=list(ports[identity]),
                 outputs=[c["id"] for c in rows if c["producer"] == identity and not c["workspace"]],
                 workspace_copies=[c["id"] for c in rows if c["producer"] == identity and c["workspace"]],
                 state_effect=any(identity in chain for chain in p.state_chains))
        events.append(e)
    events.sort(key=lambda e: (e["start"], e["id"]))
    r = dict(status=status, ordering_unit="source_steps", time_unit="source_steps",
             objective_unit=p.provenance["objective_unit"], objective=None, best_bound=None, finish_step=finish,
             optimality_certified=complete, events=events, copies=rows, output_states=[],
             profiles=json.loads(json.dumps(dict(p.profiles))), provenance=dict(p.provenance),
             model_sha256=hashlib.sha256(json.dumps(problem_to_dict(p), sort_keys=True).encode()).hexdigest(),
             solver="depth-first branch and bound over source orders (no external solver)")
    r["actions"] = r["events"]
    r["output_states"] = [dict(stripe=s, tier="reg", bytes=OUTPUT_STRIPE_BYTES, start=step_of[chain[0]],
                               end=step_of[chain[-1]] + 1, first_event=chain[0], last_event=chain[-1],
                               effect_order=list(chain)) for s, chain in enumerate(p.state_chains)]
    r["source_features"] = source_feature_values(p, r)
    r["lowering_trace"] = lowering_trace(p, r)
    r["cp_lowering_frontier"] = None  # the frontier certificate belongs to a constraint model; there is none here
    r["objective"] = evaluate_objective(p, r)
    r["objective_features"] = objective_features(p, r)
    r["cp_source_features"] = {json.dumps(term["source"], sort_keys=True): r["source_features"][term["source"]["kind"]]
                               for term in p.objective_spec["terms"] if "source" in term}
    r["objective_model"] = {"kind": "affine_features", "spec": p.objective_spec, "unit": p.provenance["objective_unit"]}
    return r


def objective_lower_bound(p, graph):
    """A bound no source order of the bound graph can beat, whatever the slab addresses: every selected action
    is counted; a register copy is alive at least in its producer's step and, if anything reads it, in one
    later step; an output stripe's state at least one step per action of its chain."""
    selected, _, copies, consumers, _ = graph
    rf = sum(_kib(c["occupied_bytes"]) * (2 if consumers[identity] else 1)
             for identity, c in copies.items() if c["tier"] == "reg")
    rf += sum(_kib(OUTPUT_STRIPE_BYTES) * len(chain) for chain in p.state_chains)
    floor = {"source_actions": len(selected), "rf_kib_steps": rf}
    total = p.objective_spec.get("constant", 0)
    for term in p.objective_spec["terms"]:
        require(term["coefficient"] >= 0 and _term_source(term) in floor,
                "The bound covers non-negative action-count and RF terms")
        total += term["coefficient"] * floor[_term_source(term)]
    return total


def solve(p, max_time_seconds=15, artifact_dir=None):
    """Plan one arm: bind ports, search source orders and slab offsets, replay the winner.

    Returns the reference's result dictionary (``model.py:1131-1197``). ``status`` is ``OPTIMAL`` when
    the search space was exhausted within the time budget, ``FEASIBLE`` when the best plan found so
    far is returned, ``INFEASIBLE`` / ``UNKNOWN`` otherwise. Deterministic: no randomness, ties broken
    by action identity.
    """
    validate_problem(p)
    require(0 < max_time_seconds <= 120, "Time budget must be in (0, 120] seconds")
    started = time.perf_counter()
    variants = p.plan.get("alternatives") or [{}]
    best = None
    complete = True
    floor = None
    for overrides in variants:
        graph = _bound_graph(p, overrides)
        bound = objective_lower_bound(p, graph)
        floor = bound if floor is None else min(floor, bound)
        # The budget is counted in search nodes, not seconds, so that the same call returns the same
        # plan on every machine (about 20k nodes per second of the nominal budget).
        search = _Search(p, graph, int(NODES_PER_SECOND * max_time_seconds / len(variants)))
        cost, trail = search.run()
        complete = complete and search.complete
        if trail is not None and (best is None or cost < best[0]):
            best = (cost, trail, graph)
    if best is None:
        r = dict(status="INFEASIBLE" if complete else "UNKNOWN", events=[], copies=[], output_states=[],
                 provenance=dict(p.provenance), finish_step=None, objective=None)
    else:
        # `complete` means the order space was exhausted under the slab-placement heuristic (three candidate
        # offsets per write), which proves nothing about orders that need another address: the optimum is
        # certified only when the objective meets the address-free lower bound.
        certified = complete and best[0] == floor
        r = _materialise(p, best[2], best[1], "OPTIMAL" if certified else "FEASIBLE", certified)
        require(r["objective"] == best[0], "Search cost and replayed objective differ")
        multiplier = len(p.actions) + 1
        r["best_bound"] = r["objective"] if certified else floor
        r["lexicographic_objective"] = {"combined": r["objective"] * multiplier + r["finish_step"],
                                        "combined_bound": r["best_bound"] * multiplier + (r["finish_step"] if certified else 0),
                                        "cost_multiplier": multiplier}
        r["replay"] = replay(p, r)
    r["solver_wall_seconds"] = time.perf_counter() - started
    if artifact_dir is not None:
        artifact_dir = Path(artifact_dir)
        artifact_dir.mkdir(parents=True, exist_ok=True)
        (artifact_dir / "result.json").write_text(json.dumps(r, indent=2) + "\n")
    return r


def replay(p, r):
    """Independent validation of a result: raises ``ValueError`` on the first inconsistency.

    Checks (cf. ``model.py:1205-1355``): serial unit-step timing; every event is a known action with
    its declared ports bound to copies of the right value and tier that were produced earlier; copy
    lifetimes span producer start to last consumer end; shared copies are slab-aligned, inside the
    arena and never overlap while live; the register budget holds at every step; precedence edges and
    the plan's ordering relations hold; recomputed features, objective and lowering trace equal the
    stored ones; and the residency contract's own verifier accepts the plan.
    """
    require(r.get("status") in ("OPTIMAL", "FEASIBLE"), "Replay needs a solved plan")
    actions = {a["id"]: a for a in p.actions}
    events = {e["id"]: e for e in r["events"]}
    copies = {c["id"]: c for c in r["copies"]}
    require(len(events) == len(r["events"]) and len(copies) == len(r["copies"]), "Duplicate event or copy identities")
    require(sorted(e["start"] for e in r["events"]) == list(range(len(events)))
            and all(e["end"] == e["start"] + 1 for e in r["events"]) and r["finish_step"] == len(events),
            "Events must occupy consecutive unit source steps")
    require({a["id"] for a in p.actions if a["mandatory"]} <= set(events), "A mandatory action is missing")
    for e in r["events"]:
        require(e["id"] in actions and actions[e["id"]]["kind"] == e["kind"], f"Unknown event {e['id']}")
        ports = actions[e["id"]]["input_refs"]
        require(len(ports) == len(e["inputs"]), f"{e['id']} must bind every input port")
        require(all(e[k] == actions[e["id"]][k] for k in ("profile_key", "profile_cost", "duration")),
                f"{e['id']} changed its declared cost record")
        for (name, tier), source in zip(ports, e["inputs"]):
            require(source in copies, f"{e['id']} reads unknown copy {source}")
            c = copies[source]
            require(c["value"] == name and c["tier"] == tier, f"{e['id']} reads {source} of the wrong value or tier")
            require(c["available"] <= e["start"] and e["end"] <= c["end"], f"{e['id']} reads {source} outside its lifetime")
        produced = [c["id"] for c in r["copies"] if c["producer"] == e["id"] and not c["workspace"]]
        require(sorted(produced) == sorted(e["outputs"]) and len(produced) == len(actions[e["id"]]["output_refs"]),
                f"{e['id']} outputs disagree with its copies")
    consumers = {identity: [e for e in r["events"] if identity in e["inputs"]] for identity in copies}
    inputs_wanted = {"gmem:" + v.name for v in p.values if v.role in ("q", "k", "v")}
    require({c["id"] for c in r["copies"] if c["producer"] is None} == inputs_wanted, "Kernel inputs invented or missing")
    for c in r["copies"]:
        if c["producer"] is None:
            require(c["tier"] == "gmem" and c["id"] == "gmem:" + c["value"] and c["start"] == c["available"] == 0
                    and c["end"] == r["finish_step"] and c["offset_bytes"] is None, f"{c['id']} is not a kernel input")
            continue
        producer = events.get(c["producer"])
        require(producer is not None and c["start"] == producer["start"] and c["available"] == producer["end"],
                f"{c['id']} lifetime does not start at its producer")
        last = max([e["end"] for e in consumers[c["id"]]] or [c["available"]])
        require(c["end"] == last, f"{c['id']} lifetime does not end at its last consumer")
        if c["tier"] == "smem":
            require(integer(c["offset_bytes"]) and c["offset_bytes"] % SLAB_BYTES == 0
                    and c["occupied_bytes"] % SLAB_BYTES == 0 and c["occupied_bytes"] >= c["logical_bytes"]
                    and c["offset_bytes"] + c["occupied_bytes"] <= p.arena_slabs * SLAB_BYTES,
                    f"{c['id']} has an invalid arena span")
    shared = [c for c in r["copies"] if c["tier"] == "smem"]
    for i, a in enumerate(shared):
        for b in shared[:i]:
            if max(a["start"], b["start"]) < min(a["end"], b["end"]):
                require(a["offset_bytes"] + a["occupied_bytes"] <= b["offset_bytes"]
                        or b["offset_bytes"] + b["occupied_bytes"] <= a["offset_bytes"],
                        f"Live shared copies {a['id']} and {b['id']} overlap")
    for a, b, *gap in [*p.precedence_edges, *p.plan.get("before", ())]:
        if a in events and b in events:
            require(events[a]["end"] + (gap[0] if gap else 0) <= events[b]["start"], f"{a} must precede {b}")
    require(len(r["output_states"]) == len(p.state_chains), "One output state per stripe")
    for state, chain in zip(r["output_states"], p.state_chains):
        require(state["start"] == events[chain[0]]["start"] and state["end"] == events[chain[-1]]["end"]
                and state["bytes"] == OUTPUT_STRIPE_BYTES, "Output state lifetime differs from its chain")
    peak = 0
    for step in range(r["finish_step"]):
        live = sum(c["occupied_bytes"] for c in r["copies"] if c["tier"] == "reg" and c["start"] <= step < c["end"])
        live += sum(s["bytes"] for s in r["output_states"] if s["start"] <= step < s["end"])
        require(live <= p.register_budget_bytes, f"Register budget exceeded at step {step}")
        peak = max(peak, live)
    require(r["profiles"] == json.loads(json.dumps(dict(p.profiles))) and r["provenance"] == dict(p.provenance),
            "Cost records or provenance differ from the problem's")
    require(integer(r["best_bound"]) and r["best_bound"] <= r["objective"] and isinstance(r["optimality_certified"], bool)
            and (not r["optimality_certified"] or r["best_bound"] == r["objective"]), "Invalid objective bound")
    lex = r["lexicographic_objective"]
    require(lex["cost_multiplier"] == len(p.actions) + 1
            and lex["combined"] == r["objective"] * lex["cost_multiplier"] + r["finish_step"]
            and lex["combined_bound"] <= lex["combined"], "Invalid lexicographic objective record")
    require(r["objective_features"] == objective_features(p, r), "Stored objective features differ from the plan")
    require(r["source_features"] == source_feature_values(p, r), "Stored source features differ from the plan")
    require(r["objective"] == evaluate_objective(p, r), "Stored objective differs from the plan")
    require(r["lowering_trace"] == lowering_trace(p, r), "Stored lowering trace differs from the plan")
    peak_shared = max(sum(c["occupied_bytes"] for c in shared if c["start"] <= step < c["end"])
                      for step in range(r["finish_step"]))
    executions = {}
    for e in sorted(r["events"], key=lambda e: e["start"]):
        executions[e["name"]] = executions.get(e["name"], 0) + 1
    # peak_bytes / executions / source_order_steps / objective are the quantities the reference's replay
    # reports (model.py:1346-1355), so that the two replays can be compared field by field.
    summary = {"valid": True, "events": len(events), "peak_register_bytes": peak,
               "peak_bytes": {"reg": peak, "smem": peak_shared}, "executions": executions,
               "q_global_loads": executions.get("copy_Q", 0), "source_order_steps": r["finish_step"],
               "objective": r["objective"], "objective_unit": r["objective_unit"],
               "objective_features": r["objective_features"],
               "shared_high_water_bytes": max(c["offset_bytes"] + c["occupied_bytes"] for c in shared)}
    if p.plan.get("contract"):
        from . import exchange

        summary["residency_certificate"] = exchange.verify(p.plan["contract"], r)
    return summary

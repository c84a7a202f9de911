"""Lower a solved two-tile plan to straight-line sm_100a CUDA plus a manifest.

Counterpart of ``tilecadence/emit_exchange.py`` (``validate`` :42-83, ``source_for`` :86-406,
``emit`` :409-421). Generation runs on the CPU and imports neither torch nor CUDA. Events are walked
in start order and each becomes one call into ``csrc/exchange/backend.cuh``; a CTA release is emitted
only where a shared write lands on a slab with distributed reads outstanding, and a copy wait only
where the producing copy is newer than the ready cutoff. Both are re-derived here from the events and
byte spans and compared with the planner's lowering oracle row by row; a disagreement aborts the
emission. The emitted ``plan.cu`` also carries the host launcher and the C-ABI entry points
(``tc_exchange_forward_out``, ``tc_exchange_resources``).
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
import shutil

from . import model
from .cuda_runtime import staged_sources

SLAB = model.SLAB_BYTES
ALLOWED = set(model.ACTION_KINDS)
RESOURCE_KEYS = ("block_m", "block_n", "head_dim", "value_stripe_dim", "threads", "dynamic_shared_bytes",
                 "static_shared_bytes", "registers_per_thread", "local_bytes_per_thread", "binary_version",
                 "ptx_version", "theoretical_active_ctas_per_sm", "required_nonce_elements", "diagnostic_guard")


INDENT = "    "  # generated statements sit one level inside the kernel body


def _mapping(value):
    if isinstance(value, (str, Path)):
        return json.loads(Path(value).read_text())
    if isinstance(value, model.Problem):
        return model.problem_to_dict(value)
    return dict(value)


def validate(problem, result):
    """Replay the plan and check that it fits this backend's fixed geometry."""
    p, r = _mapping(problem), _mapping(result)
    typed = model.problem_from_dict(p)
    checked = model.replay(typed, r)
    if typed.provenance.get("shape") != model.SHAPE:
        raise ValueError("The sm_100a backend is fixed to M64/N32/D128 with two 64-wide output stripes")
    sizes = {"q": 16384, "k": 8192, "v": 4096, "p": 4096, "workspace": 8192}
    copies = {c["id"]: dict(c) for c in r["copies"]}
    for c in copies.values():
        if c["tier"] == "smem" and c["occupied_bytes"] != sizes.get(c["role"]):
            raise ValueError(f"Unexpected shared footprint for {c['id']}")
    events = sorted(r["events"], key=lambda e: (e["start"], e["id"]))
    if any(e["kind"] not in ALLOWED for e in events):
        raise ValueError("Unsupported action kind")
    if {s["stripe"] for s in r["output_states"]} != {0, 1}:
        raise ValueError("Both output stripes are required")
    for e in events:
        work = [copies[x] for x in e.get("workspace_copies", [])]
        if e["kind"] == "normalize_store":
            if len(work) != 1 or work[0]["start"] != e["start"] or work[0]["end"] != e["end"]:
                raise ValueError("The close needs one scratch span scoped to its own step")
        elif work:
            raise ValueError("Only the close has shared scratch")
    return p, r, typed, copies, events, checked


def source_for(problem, result, *, output_cache="default"):
    """Return (CUDA source, manifest) without compiling or launching anything."""
    if output_cache not in ("default", "streaming_cs"):
        raise ValueError("Declare an explicit output cache policy")
    p, r, typed, copies, events, checked = validate(problem, result)
    names = {identity: f"r{i}" for i, identity in enumerate(copies)}
    smem = {identity: f"s{i}" for i, identity in enumerate(copies)
            if copies[identity]["tier"] == "smem" and not copies[identity].get("workspace")}
    lines = [
        "// Generated from planner events, concrete copy bindings and shared byte offsets: do not edit.",
        "// Complete attention for 64 queries x 64 keys, D128, two 64-wide output stripes, one CTA per (batch, head).",
        f"#define TC_EXCHANGE_OUTPUT_STREAMING_STORE {int(output_cache == 'streaming_cs')}",
        '#include "backend.cuh"',
        '#include "tc_host.cuh"',
        "",
        "namespace {",
        "using namespace tc_exchange;",
        "template <class Element, bool Causal>",
        "__global__ void __launch_bounds__(128) solver_attention(const __grid_constant__ CUtensorMap qmap,",
        "    const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, Element* O, float* LSE,",
        "    int H, int32_t* status) {",
        "    static_assert(sizeof(Element) == 2);",
        "    extern __shared__ unsigned char arena_raw[];",
        "    unsigned char* arena = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(arena_raw) + 1023) & ~uintptr_t(1023));",
        "    __shared__ uint64_t barriers[kMaxCopies];",
        "    const Context ctx = make_context(arena, barriers, status);",
        "    const int row_stride = H * 128;",
        "    Element* o_base = O + (int64_t(ctx.batch) * 64 * H + ctx.head) * 128;",
        "    float* lse_base = LSE + (int64_t(ctx.batch) * H + ctx.head) * 64;",
    ]
    for identity, name in smem.items():
        c = copies[identity]
        if c["role"] == "p":
            lines.append(f"    Element* {name}=reinterpret_cast<Element*>(arena+{c['offset_bytes']});")
        else:
            lines.append(f"    unsigned char* {name}=arena+{c['offset_bytes']};")
    event_lines, primitives = {}, {}
    unreleased = []           # [(copy id, (lo, hi))] distributed shared reads not yet followed by a CTA barrier
    issued = waited = 0       # copies issued / covered by a wait so far
    max_pending = 0
    ready_cutoff = 0
    hmma_gap = ex2_gap = 0
    opened = set()
    by_event = {e["id"]: e for e in events}
    oracle = {row["id"]: row for row in r["lowering_trace"]}

    def span(c):
        return (c["offset_bytes"], c["offset_bytes"] + c["occupied_bytes"])

    def read_mask():
        mask = 0
        for _, (lo, hi) in unreleased:
            mask |= ((1 << ((hi - lo) // SLAB)) - 1) << (lo // SLAB)
        return mask

    def write(statement):
        lines.append(INDENT + statement)

    for event in events:
        kind = event["kind"]
        consumed = [copies[identity] for identity in event["inputs"] if copies[identity]["tier"] != "gmem"]
        produced = [copies[identity] for identity in event["outputs"]]
        ins = [names[copy["id"]] for copy in consumed]
        outs = [names[copy["id"]] for copy in produced]
        event_lines[event["id"]] = {"comment_line": len(lines) + 1}
        write("// EVENT " + event["id"])
        entry = {"kind": kind, "workspace_copies": event.get("workspace_copies", []), "read_mask_before": read_mask(),
                 "ready_cutoff_before": ready_cutoff, "last_commit_hmma_before": hmma_gap,
                 "last_commit_ex2_before": ex2_gap, "wait_before_load": False, "acquire_before_load": False}
        writes = [c for c in produced if c["tier"] == "smem"] if kind in ("copy_g2s", "store_r2s") else []
        if kind == "normalize_store":
            writes = [copies[x] for x in event["workspace_copies"]]
        hazards = [[c["id"], old] for c in writes for old, (lo, hi) in unreleased if span(c)[0] < hi and lo < span(c)[1]]
        if hazards:
            write("release_shared_reads();  // this shared write overlaps slabs with distributed reads outstanding")
            unreleased.clear()
        entry.update(release_before_write=bool(hazards), shared_read_write_hazards=hazards)
        if kind == "copy_g2s":
            dst = produced[0]
            role, tile, stripe = dst["role"], dst["tile"], dst["stripe"]
            if issued >= 16:
                raise ValueError("More copies than the kernel has barriers for")
            if role == "q":
                write(f"issue_g2s<Element,64,128,{issued}>(ctx,&qmap,0,0,{smem[dst['id']]});")
            elif role == "k":
                write(f"issue_g2s<Element,32,128,{issued}>(ctx,&kmap,{tile * 32},0,{smem[dst['id']]});")
            elif role == "v" and stripe is not None:
                write(f"issue_g2s<Element,32,64,{issued}>(ctx,&vmap,{tile * 32},{stripe * 64},{smem[dst['id']]});")
            else:
                raise ValueError("Only Q, K and V stripes have global copies")
            entry.update(primitive="tma_tile_copy_arm_mbarrier", barrier_index=issued)
            issued += 1
            max_pending = max(max_pending, issued - waited)
            if issued - waited > model.MAX_OUTSTANDING_COPIES:
                raise ValueError("More than eight copies in flight")
        elif kind == "load_s2r":
            src, dst = consumed[0], produced[0]
            role = dst["role"]
            producer = by_event[src["producer"]]
            wait = False
            if role == "p":
                if producer["kind"] != "store_r2s":
                    raise ValueError("A checkpoint load needs its checkpoint store")
                write(f"auto {outs[0]}=load_checkpoint<Element>({smem[src['id']]},ctx);")
                entry.update(primitive="load_checkpoint")
            else:
                if producer["kind"] != "copy_g2s":
                    raise ValueError("An operand load needs its input copy")
                wait = producer["end"] > ready_cutoff
                if wait:
                    write(f"acquire_copies<{waited},{issued}>(ctx);  // copy newer than the ready cutoff")
                    unreleased.clear()
                    waited, ready_cutoff = issued, event["end"]
                loader = {"q": "load_q_ready", "k": "load_k_ready", "v": "load_v_ready"}[role]
                write(f"auto {outs[0]}={loader}<Element>(ctx,{smem[src['id']]});")
                entry.update(primitive="ldmatrix_after_acquire" if wait else "ldmatrix_ready")
            if src["id"] not in [identity for identity, _ in unreleased]:
                unreleased.append((src["id"], span(src)))
            entry.update(wait_before_load=wait, acquire_before_load=wait)
        elif kind == "store_r2s":
            write(f"store_checkpoint({ins[0]},{smem[produced[0]['id']]},ctx);")
            unreleased.clear()  # store_checkpoint ends with a CTA barrier
            entry.update(primitive="store_checkpoint_with_cta_barrier")
        elif kind == "qk":
            write(f"auto {outs[0]}=qk<Element>({ins[0]},{ins[1]});")
        elif kind in ("stats_first", "stats_next"):
            for c, name in zip(produced, outs):
                write(f"Probabilities<Element> {name};" if c["role"] == "p" else f"RowPair {name};")
            tile = event["tile"]
            if kind == "stats_first":
                write(f"stats_first<Causal,{tile},Element>(ctx,{ins[0]},{outs[0]},{outs[1]},{outs[2]});")
            else:
                write(f"stats_next<Causal,{tile},Element>(ctx,{ins[0]},{ins[1]},{ins[2]},{outs[0]},{outs[1]},{outs[2]},{outs[3]});")
        elif kind in ("pv_first", "pv_next"):
            stripe = event["stripe"]
            if kind == "pv_first":
                if stripe in opened:
                    raise ValueError("An output stripe may only be opened once")
                write(f"Accumulator o{stripe};")
                write(f"clear(o{stripe});  // the stripe's register lifetime begins here")
                opened.add(stripe)
            elif stripe not in opened:
                raise ValueError("PV update before the stripe was opened")
            write(f"pv<Element>({ins[0]},{ins[1]},o{stripe});")
        elif kind == "rescale_o":
            write(f"rescale(o{event['stripe']},{ins[0]});")
        elif kind == "normalize_store":
            stripe = event["stripe"]
            scratch = copies[event["workspace_copies"][0]]
            write(f"normalize_store_coalesced128<Element,{stripe}>(ctx,o{stripe},{ins[0]},o_base,row_stride,arena+{scratch['offset_bytes']});")
            entry.update(primitive="close_shared128", scratch_offset_bytes=scratch["offset_bytes"], scratch_bytes=8192)
            unreleased.clear()  # the close has a CTA barrier between its shared writes and reads
            unreleased.append((scratch["id"], span(scratch)))
        elif kind == "store_lse":
            write(f"store_lse(ctx,{ins[0]},{ins[1]},lse_base);")
        else:
            raise ValueError("Unsupported action")
        event_lines[event["id"]]["last_line"] = len(lines)
        wait = entry["wait_before_load"]
        entry.update(last_commit_wait_hmma_sites=hmma_gap if wait else 0, last_commit_wait_ex2_sites=ex2_gap if wait else 0)
        if kind == "copy_g2s" or wait:
            hmma_gap = ex2_gap = 0
        else:
            hmma, ex2 = model.MATH_SITE_WEIGHTS.get(kind, (0, 0))
            hmma_gap, ex2_gap = hmma_gap + hmma, ex2_gap + ex2
        entry.update(last_commit_hmma_after=hmma_gap, last_commit_ex2_after=ex2_gap, read_mask_after=read_mask(),
                     ready_cutoff_after=ready_cutoff, pending_copies_after=issued - waited)
        expected = oracle[event["id"]]
        keys = ("read_mask_before", "read_mask_after", "ready_cutoff_before", "ready_cutoff_after", "wait_before_load",
                "acquire_before_load", "release_before_write", "shared_read_write_hazards", "last_commit_hmma_before",
                "last_commit_hmma_after", "last_commit_ex2_before", "last_commit_ex2_after",
                "last_commit_wait_hmma_sites", "last_commit_wait_ex2_sites")
        if any(entry[key] != expected[key] for key in keys):
            raise ValueError("Independent CUDA lowering differs from the ready/mask certificate at " + event["id"])
        if issued - waited != expected["issued_groups_after"] - expected["ready_groups_after"]:
            raise ValueError("Issued/observed copy certificate differs at " + event["id"])
        primitives[event["id"]] = entry
    arena_bytes = typed.arena_slabs * SLAB
    if max(c["offset_bytes"] + c["occupied_bytes"] for c in copies.values() if c["tier"] == "smem") > arena_bytes:
        raise ValueError("Copy or scratch spans exceed the declared arena")
    lines.append("}")
    lines.extend(_HOST_TEMPLATE.replace("@ARENA@", str(arena_bytes)).splitlines())
    source = "\n".join(lines) + "\n"
    manifest = {
        "schema": "tilecadence-b200-exchange-manifest-v1",
        "target": "sm_100a",
        "contract": typed.plan.get("contract"),
        "arena_bytes": arena_bytes,
        "dynamic_shared_bytes": arena_bytes + 1024,
        "threads": 128,
        "copies_issued": issued,
        "max_copies_in_flight": max_pending,
        "event_source_lines": event_lines,
        "primitives": primitives,
        "source_ready_mask_certificate": r["lowering_trace"],
        "replay": checked,
        "resource_keys": list(RESOURCE_KEYS),
        "output_cache": output_cache,
        "plan_sha256": hashlib.sha256(source.encode()).hexdigest(),
    }
    return source, manifest


def emit(problem, result, out, **options):
    """Write ``plan.cu``, the backend and host headers and ``manifest.json`` into a new directory."""
    source, manifest = source_for(problem, result, **options)
    out = Path(out)
    out.mkdir(parents=True, exist_ok=False)
    for name, path in staged_sources("exchange").items():
        if name != "plan.cu":
            shutil.copyfile(path, out / name)
    (out / "plan.cu").write_text(source, encoding="utf-8", newline="\n")
    (out / "manifest.json").write_text(json.dumps(manifest, indent=2) + "\n", encoding="utf-8")
    return manifest


_HOST_TEMPLATE = r'''
constexpr int kArenaBytes = @ARENA@;
constexpr int kDynamicShared = kArenaBytes + 1024;  // slack for the 1024-byte alignment of the arena

template <class Element, bool Causal>
int launch(const CUtensorMap& qmap, const CUtensorMap& kmap, const CUtensorMap& vmap, void* out, float* lse,
           int64_t batch, int64_t heads, int32_t* status, cudaStream_t stream) {
    auto kernel = &solver_attention<Element, Causal>;
    TC_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDynamicShared));
    kernel<<<dim3(1, unsigned(batch), unsigned(heads)), 128, kDynamicShared, stream>>>(
        qmap, kmap, vmap, static_cast<Element*>(out), lse, int(heads), status);
    TC_CUDA(cudaGetLastError());
    return TC_OK;
}

template <class Element, bool Causal>
int describe(int64_t* values) {
    int64_t attributes[8];
    int status = tc::kernel_resources(&solver_attention<Element, Causal>, 128, kDynamicShared, attributes);
    if (status != TC_OK) return status;
    const int64_t row[14] = {64, 32, 128, 64, attributes[0], attributes[1], attributes[2], attributes[3],
                             attributes[4], attributes[5], attributes[6], attributes[7], 0, 0};
    for (int i = 0; i < 14; ++i) values[i] = row[i];
    return TC_OK;
}

}  // namespace

extern "C" {

int tc_exchange_forward_out(int device, void* stream, const void* q, const void* k, const void* v, void* out,
                            float* lse, int64_t batch, int64_t heads, int dtype_fp16, int causal) {
    tc::DeviceInfo info;
    int status = tc::require_sm100(device, &info);
    if (status != TC_OK) return status;
    TC_REQUIRE(q && k && v && out && lse, "null tensor pointer");
    TC_REQUIRE(batch > 0 && batch <= 65535 && heads > 0 && heads <= 65535, "B and H must be positive and fit the CUDA grid");
    const size_t bytes = size_t(batch) * 64 * heads * 128 * 2, lse_bytes = size_t(batch) * heads * 64 * 4;
    for (const void* pointer : {q, k, v, static_cast<const void*>(out)})
        TC_REQUIRE(reinterpret_cast<uintptr_t>(pointer) % 16 == 0, "16-byte aligned Q/K/V/O required");
    for (const void* input : {q, k, v})
        TC_REQUIRE(!tc::ranges_overlap(out, bytes, input, bytes) && !tc::ranges_overlap(lse, lse_bytes, input, bytes),
                   "Outputs may not alias inputs");
    TC_REQUIRE(!tc::ranges_overlap(out, bytes, lse, lse_bytes), "Outputs may not alias each other");
    tc::DeviceGuard guard(device);
    TC_CUDA(guard.status);
    tc::DeviceScratch scratch;
    if ((status = tc::device_scratch(device, &scratch)) != TC_OK) return status;
    CUtensorMap qmap, kmap, vmap;
    const bool fp16 = dtype_fp16 != 0;
    if ((status = tc::make_rows_map(&qmap, q, fp16, heads, 64, batch, 128, heads * 128, 64 * heads * 128, 64, 2)) != TC_OK) return status;
    if ((status = tc::make_rows_map(&kmap, k, fp16, heads, 64, batch, 128, heads * 128, 64 * heads * 128, 32, 2)) != TC_OK) return status;
    if ((status = tc::make_rows_map(&vmap, v, fp16, heads, 64, batch, 128, heads * 128, 64 * heads * 128, 32, 2)) != TC_OK) return status;
    const cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (fp16)
        return causal ? launch<__half, true>(qmap, kmap, vmap, out, lse, batch, heads, scratch.status, s)
                      : launch<__half, false>(qmap, kmap, vmap, out, lse, batch, heads, scratch.status, s);
    return causal ? launch<__nv_bfloat16, true>(qmap, kmap, vmap, out, lse, batch, heads, scratch.status, s)
                  : launch<__nv_bfloat16, false>(qmap, kmap, vmap, out, lse, batch, heads, scratch.status, s);
}

int tc_exchange_resources(int device, int dtype_fp16, int causal, int64_t values[14]) {
    tc::DeviceInfo info;
    int status = tc::require_sm100(device, &info);
    if (status != TC_OK) return status;
    TC_REQUIRE(values, "null values");
    tc::DeviceGuard guard(device);
    TC_CUDA(guard.status);
    if (dtype_fp16) return causal ? describe<__half, true>(values) : describe<__half, false>(values);
    return causal ? describe<__nv_bfloat16, true>(values) : describe<__nv_bfloat16, false>(values);
}

}  // extern "C"
'''

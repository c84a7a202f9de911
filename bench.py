"""Benchmark of the B200 attention hot path: causal GQA prefill (headline) and split-KV decode.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

For N > 1 launch with ``python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N``.
Rank 0 prints ONE JSON line.

Headline workload (``config.workload``): BASELINE config 2, causal prefill, BF16, batch 1, 8192
tokens, 32 query / 8 KV heads, D = 128, N(0,1) inputs from seed 1 (synthetic stand-ins for the
reference's saved Qwen3 projections). A step is one forward over that batch.

* ``value``      TFLOP/s (4*B*Hq*S^2*D/2 per step) with inputs resident in HBM. At N > 1 that ONE batch is
                 split by KV-head group over the ranks (rank r holds KV heads [8r/N, 8(r+1)/N) and their
                 query heads; no collective): strong scaling, value = the batch's FLOPs / the slowest rank's
                 time. ``prefill_replicas`` (N > 1) is the other experiment, one whole batch per rank.
* ``e2e``        the same metric through the operator API with HOST buffers: every step copies its
                 (slice of) Q/K/V from pinned host memory and reads O and LSE back; copies and kernels of
                 neighbouring steps overlap on four streams (two uploads, compute, download).
* ``roofline``   the prefill kernel against the measured dense BF16 peak.
* ``decode``     split-KV decode with fused append: config 4 (batch 1, 8192 of 32768 rows valid) and
                 config 5 (batch 4, 32768 rows attended; KV sequence sharded over the ranks when N > 1 and
                 merged inside the decode launch over NVLink, with the all-gather + combine route beside
                 it as ``c5_nccl``), as HBM GB/s with their own roofline.
* ``project``    the step before decode (fused QKV projection + head RMS norm + RoPE, 4 tokens, Qwen3-4B
                 shapes) as HBM GB/s of streamed weights.
* ``layer_chain`` projection then config-4 decode as a layer runs them, microseconds per layer, with the plain
                 decode entry and with the cache-stable promise (K/V streamed while the projection finishes).
* ``checks``     (N > 1) results of the sharded paths compared outside the timed regions: the sharded prefill
                 against the CPU oracle on sampled rows, both sharded decode routes bit for bit against the
                 standalone combine of the same shards' partials and against the CPU oracle on sampled heads.
                 A miss ends the run with a non-zero exit code.
* ``cpu_baseline`` the CPU oracle (the reference's only CPU attention, ``bench_exchange.py:54-60``)
                 timed on this host on a bounded sample.

``--impl reference`` times that CPU attention alone on the whole config-2 batch, on rank 0, with all host
threads.
"""
from __future__ import annotations

import argparse
import json
import os
from pathlib import Path
import statistics
import subprocess
import sys
import time

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the three benchmarked launches, from
# the ncu captures summarised under profiles/.
NCU_TRAFFIC_BYTES = {"prefill_c2": 119.5e6, "decode_c4": 33.62e6, "decode_c5": 541.2e6, "project": 31.5e6}
HQ, HKV, DIM = 32, 8, 128
SCALE = DIM ** -0.5
PREFILL = dict(batch=1, tokens=8192, seed=1)
DECODE_C4 = dict(batch=1, capacity=32768, valid=8192, seed=3)
DECODE_C5 = dict(batch=4, capacity=32768, valid=32767, seed=4)
METRIC = "causal_prefill_tflops"
UNIT = "TFLOP/s"
WORKLOAD = "config2 causal GQA prefill B1 S8192 Hq32 Hkv8 D128 seed1"


def prefill_flops(batch, tokens, heads=HQ):
    return 4.0 * batch * heads * tokens * tokens * DIM / 2.0


def decode_bytes(batch, attended, kv_heads=HKV):
    """Algorithmic HBM bytes of one decode step: K and V rows attended, Q in, O out, LSE, new rows in + out."""
    q_heads = kv_heads * 4
    return (2 * batch * attended * kv_heads * DIM * 2 + 2 * batch * q_heads * DIM * 2 + batch * q_heads * 4
            + 4 * batch * kv_heads * DIM * 2)


def prefill_rank_bytes(world):
    """Bytes of one rank's Q, K, V, O and LSE for its KV-head-group share of the headline batch."""
    batch, tokens = PREFILL["batch"], PREFILL["tokens"]
    heads_q, heads_kv = HQ // world, HKV // world
    return batch * tokens * ((2 * heads_q + 2 * heads_kv) * DIM * 2 + heads_q * 4)


def prefill_buffer_sets(world):
    """Rotating buffer sets per rank: a shard smaller than L2 would be re-read from L2 by the next step, so enough
    sets rotate that a set is evicted before its turn comes again. One rank's whole batch (169 MB) exceeds L2."""
    rank_bytes = prefill_rank_bytes(world)
    return 1 if rank_bytes > 130e6 else -(-int(2.2 * 126e6) // rank_bytes)


def bench_config(world):
    """The ``config`` object of the JSON line: both arms state the same workload."""
    if world == 1:
        return {"workload": WORKLOAD + ", one GPU",
                "l2": "inputs+outputs 161 MiB per step, larger than the 126 MB L2",
                "decode_l2": "rotating cache sets larger than L2",
                "timing": "direct operator calls back to back"}
    return {"workload": WORKLOAD + f", the one batch split by KV-head group over {world} GPUs ({HKV // world} KV / "
                        f"{HQ // world} query heads per GPU, no collective)",
            "l2": f"{prefill_buffer_sets(world)} rotating buffer sets of {prefill_rank_bytes(world) / 2**20:.0f} MiB per "
                  "GPU, together larger than twice the 126 MB L2",
            "decode_l2": "rotating cache sets larger than L2",
            "timing": "one captured graph per buffer set, replayed back to back"}


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        data = json.loads(path.read_text())
        return dict(hbm=data["hbm_gbs"], bf16=data["bf16_tflops"], bf16_sustained=data["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid):
        self.uuid, self.process, self.rows = uuid, None, []

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", self.uuid, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None
        return self

    def __exit__(self, *exc):
        if self.process is not None:
            time.sleep(0.15)
            self.process.terminate()
            try:
                output, _ = self.process.communicate(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()
                output, _ = self.process.communicate()
            for line in output.splitlines():
                parts = [part.strip() for part in line.split(",")]
                if len(parts) == 7:
                    self.rows.append(parts)

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        clocks = [float(row[0]) for row in self.rows if row[0].replace(".", "").isdigit()]
        busy = [c for c in clocks if c > 0.5 * max(clocks)] or clocks
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [name for index, name in enumerate(names) if any(row[3 + index] == "Active" for row in self.rows)]
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": float(self.rows[0][1]), "reasons": reasons,
                "samples": len(self.rows)}


# --------------------------------------------------------------------------------------- CPU arm
def cpu_attention_sample(torch, oracle, seconds_hint=10.0, steps=None, warmup=0, kv_groups=1):
    """Time the CPU oracle on `kv_groups` KV-head groups (4 query heads each) of the headline workload;
    8 groups is the whole config-2 batch.

    Returns (TFLOP/s, threads, description, seconds per pass). Throughput is per FLOP, so a sample of
    fewer groups needs no scaling.
    """
    from tilecadence_b200.synthetic import seeded_normal

    torch.set_num_threads(os.cpu_count() or 1)
    tokens = PREFILL["tokens"]
    q, k, v = seeded_normal(PREFILL["seed"], (1, tokens, HQ, DIM), (1, tokens, HKV, DIM), (1, tokens, HKV, DIM))
    q, k, v = q[:, :, :4 * kv_groups].contiguous(), k[:, :, :kv_groups].contiguous(), v[:, :, :kv_groups].contiguous()
    flops = prefill_flops(1, tokens, heads=4 * kv_groups)
    oracle.attention(q[:, :1024], k[:, :1024], v[:, :1024], causal=True)  # warm the thread pool
    for _ in range(warmup):
        oracle.attention(q, k, v, causal=True)
    times = []
    started = time.perf_counter()
    while True:
        t0 = time.perf_counter()
        oracle.attention(q, k, v, causal=True)
        times.append(time.perf_counter() - t0)
        if steps is not None:
            if len(times) >= steps:
                break
        elif time.perf_counter() - started > seconds_hint or len(times) >= 50:
            break
    best = statistics.median(times)
    what = "the whole config-2 prefill batch (32 query / 8 KV heads" if kv_groups == HKV else \
        f"{kv_groups} KV-head group(s) ({4 * kv_groups} of 32 query heads"
    description = f"{what}, all {tokens} rows), {len(times)} passes, median"
    return flops / best / 1e12, torch.get_num_threads(), description, best


def run_reference(args, rank):
    if rank != 0:
        return
    import torch
    from oracle import attention as oracle

    # The whole batch per step (about 1.6 s on 16 threads), so that this arm runs the config it states.
    value, threads, description, seconds = cpu_attention_sample(torch, oracle, steps=max(1, args.steps),
                                                                warmup=args.warmup, kv_groups=HKV)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": description + "; fp32 torch attention restating the reference's "
                                   "bench_exchange._reference, host threads only, rank 0"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------- GPU arm
def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from oracle import attention as oracle  # the checker (N > 1 result checks) and the timed CPU baseline leg
    from tilecadence_b200 import cuda_runtime, sharding
    from tilecadence_b200.synthetic import seeded_normal

    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    # Libraries (NCCL's version banner, for one) write to file descriptor 1; the contract is ONE JSON line
    # on stdout, so everything but that line is sent to stderr.
    sys.stdout.flush()
    json_out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    library = cuda_runtime.default_library()
    decode_ops = cuda_runtime.ops_for(library, "decode")
    peaks = measured_peaks()
    launches = 0

    def barrier():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def max_over_ranks(value):
        if world == 1:
            return value
        tensor = torch.tensor([value], device=device, dtype=torch.float64)
        dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
        return tensor.item()

    def timed(step, steps, warmup):
        """Milliseconds for exactly `steps` calls on the current stream, max over ranks."""
        for _ in range(warmup):
            step()
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            step()
        end.record()
        barrier()
        return max_over_ranks(start.elapsed_time(end))

    check_failures = []

    def checked(name, fn):
        """Run a result check outside the timed regions; a miss is recorded and ends the run at the end."""
        try:
            return fn()
        except AssertionError as error:
            check_failures.append(f"rank {rank}: {name}: {error}")
            print(f"CHECK FAILED on rank {rank}: {name}: {error}", file=sys.stderr, flush=True)
            return None

    def graph_of(fn):
        """One call of `fn` captured as a CUDA graph (the call runs once un-captured first)."""
        stream = torch.cuda.Stream(device)
        with torch.cuda.stream(stream):
            fn()
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                fn()
        return graph

    # ------------------------------------------------------------------ prefill, resident inputs
    # The headline batch, split by KV-head group over the ranks (all of it at N = 1).
    batch, tokens = PREFILL["batch"], PREFILL["tokens"]
    if HKV % world:
        raise SystemExit(f"{HKV} KV heads do not divide over {world} ranks")
    kv_slice, q_slice = sharding.kv_head_slice(rank, world, HKV)
    local_hq = HQ // world
    whole = seeded_normal(PREFILL["seed"], (batch, tokens, HQ, DIM), (batch, tokens, HKV, DIM), (batch, tokens, HKV, DIM))
    host = [whole[0][:, :, q_slice].contiguous().pin_memory(), whole[1][:, :, kv_slice].contiguous().pin_memory(),
            whole[2][:, :, kv_slice].contiguous().pin_memory()]
    prefill_ops = cuda_runtime.ops_for(library, "prefill", q_heads=local_hq)
    empty = torch.empty(0, device=device, dtype=torch.float32)
    sets = prefill_buffer_sets(world)
    buffers = []
    for _ in range(sets):
        dq, dk, dv = (tensor.to(device) for tensor in host)
        buffers.append(dict(q=dq, k=dk, v=dv, out=torch.empty_like(dq),
                            lse=torch.empty((batch, local_hq, tokens), device=device, dtype=torch.float32)))
    split_ws = None
    if world == 1:
        def prefill_call(slot):
            prefill_ops.forward_out(slot["q"], slot["k"], slot["v"], slot["out"], slot["lse"], empty, empty, 0, 1,
                                    SCALE, True)
            return 1
    else:
        # A shard of few heads cannot fill the GPU with one CTA per query tile: the key-split entry then gives
        # every tile to two CTAs (its own choice; with one CTA per tile it is the plain kernel).
        split_ws = torch.empty(prefill_ops.key_split_workspace_bytes(buffers[0]["q"]), device=device, dtype=torch.uint8)

        def prefill_call(slot):
            return prefill_ops.key_split_forward_out(slot["q"], slot["k"], slot["v"], slot["out"], slot["lse"], split_ws,
                                                     1, SCALE, 0)
    ctas_per_query_tile = prefill_call(buffers[0])
    turn = [0]
    if world == 1:
        def prefill_step():
            prefill_call(buffers[turn[0] % sets])
            turn[0] += 1
    else:
        # A shard's step is shorter than the Python call path, so each buffer set's step is captured once and the
        # timed region replays those graphs back to back.
        graphs = [graph_of(lambda slot=slot: prefill_call(slot)) for slot in buffers]

        def prefill_step():
            graphs[turn[0] % sets].replay()
            turn[0] += 1

    uuid = str(torch.cuda.get_device_properties(device).uuid)
    uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
    sampler = ClockSampler(uuid)  # stays open over the resident and the host-buffer timed regions
    sampler.__enter__()
    prefill_ms = timed(prefill_step, args.steps, args.warmup)
    launches += args.steps
    ms_per_step = prefill_ms / args.steps
    step_flops = prefill_flops(batch, tokens)
    value = step_flops / (ms_per_step * 1e-3) / 1e12                 # the one batch, all ranks together
    achieved = step_flops / world / (ms_per_step * 1e-3) / 1e12      # the kernel on one GPU

    # ------------------------------------------------------------------ prefill, host buffers (e2e)
    host_out = [torch.empty(buffers[0]["out"].shape, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    host_lse = [torch.empty(buffers[0]["lse"].shape, dtype=torch.float32).pin_memory() for _ in range(2)]
    slots = [{name: torch.empty_like(tensor) for name, tensor in buffers[0].items()} for _ in range(2)]
    # Two upload streams (Q on one, K and V on the other): two copy engines keep the link a little fuller than one.
    copy_in, copy_in_kv, compute, copy_out = (torch.cuda.Stream(device) for _ in range(4))

    def e2e_run(steps):
        loaded = [None, None]
        computed = [None, None]
        drained = [None, None]
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(copy_in)
        copy_in_kv.wait_event(start)
        for index in range(steps):
            slot = slots[index % 2]
            uploads = []
            for stream, names in ((copy_in, "q"), (copy_in_kv, "kv")):
                with torch.cuda.stream(stream):
                    if computed[index % 2] is not None:
                        stream.wait_event(computed[index % 2])  # the kernel that read this slot is done
                    for name in names:
                        slot[name].copy_(host["qkv".index(name)], non_blocking=True)
                    uploads.append(torch.cuda.Event())
                    uploads[-1].record(stream)
            loaded[index % 2] = uploads
            with torch.cuda.stream(compute):
                for event in loaded[index % 2]:
                    compute.wait_event(event)
                if drained[index % 2] is not None:
                    compute.wait_event(drained[index % 2])  # the previous result left this slot
                prefill_call(slot)
                computed[index % 2] = torch.cuda.Event()
                computed[index % 2].record(compute)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(computed[index % 2])
                host_out[index % 2].copy_(slot["out"], non_blocking=True)
                host_lse[index % 2].copy_(slot["lse"], non_blocking=True)
                drained[index % 2] = torch.cuda.Event()
                drained[index % 2].record(copy_out)
        copy_out.wait_stream(compute)
        end.record(copy_out)
        barrier()
        return max_over_ranks(start.elapsed_time(end))

    e2e_run(min(args.warmup, 3))
    e2e_ms = e2e_run(args.steps)
    launches += args.steps
    sampler.__exit__(None, None, None)
    clocks = sampler.summary()
    e2e_value = step_flops / (e2e_ms / args.steps * 1e-3) / 1e12
    h2d_bytes = world * sum(t.numel() * t.element_size() for t in host)
    d2h_bytes = world * (host_out[0].numel() * 2 + host_lse[0].numel() * 4)

    # ------------------------------------------------------------------ the sharded prefill's result, checked
    checks = {}
    if world > 1:
        def check_prefill(got_o, got_lse, label):
            """Sampled 64-row blocks of this rank's first and last KV-head group against the CPU oracle."""
            worst = [0.0, 0.0]
            local_kv = HKV // world
            for r0 in (0, 4032, tokens - 64):
                rows = slice(r0, r0 + 64)
                for g in sorted({0, local_kv - 1}):
                    qh = host[0][0, rows, g * 4:(g + 1) * 4].float().permute(1, 0, 2)
                    scores = (qh @ host[1][0, :r0 + 64, g].float().T) * SCALE
                    scores.masked_fill_(torch.arange(r0 + 64)[None, :] > torch.arange(r0, r0 + 64)[:, None], float("-inf"))
                    want_o = (scores.softmax(-1) @ host[2][0, :r0 + 64, g].float()).permute(1, 0, 2)
                    errors = oracle.check_outputs(got_o[0, rows, g * 4:(g + 1) * 4], got_lse[0, g * 4:(g + 1) * 4, rows],
                                                  want_o, scores.logsumexp(-1))
                    worst = [max(a, b) for a, b in zip(worst, errors)]
            assert torch.isfinite(got_lse).all() and torch.isfinite(got_o.float()).all(), f"{label}: non-finite output"
            return worst

        torch.cuda.synchronize(device)
        resident = checked("sharded prefill (resident buffers)",
                           lambda: check_prefill(buffers[-1]["out"].cpu(), buffers[-1]["lse"].cpu(), "resident"))
        through_host = checked("sharded prefill (host buffers)",
                               lambda: check_prefill(host_out[(args.steps - 1) % 2], host_lse[(args.steps - 1) % 2], "e2e"))
        ok = resident is not None and through_host is not None
        worst = [max(a, b) for a, b in zip(resident, through_host)] if ok else [float("inf")] * 2
        worst = [max_over_ranks(x) for x in worst]  # every rank takes part, whatever its own outcome
        ok = all(x != float("inf") for x in worst)
        checks["prefill"] = {"checked": ok, "against": "CPU oracle, three 64-row blocks of two KV-head groups per rank, "
                                                      "resident and host-buffer results",
                             "o_max_abs": worst[0] if ok else None, "lse_rel": worst[1] if ok else None}
    del slots, host_out, host_lse, buffers, split_ws
    if world > 1:
        del graphs
    torch.cuda.empty_cache()

    # ------------------------------------------------------------------ N > 1: one whole batch per rank (replicas)
    prefill_replicas = None
    if world > 1:
        full_ops = cuda_runtime.ops_for(library, "prefill")
        fq, fk, fv = (tensor.to(device) for tensor in whole)
        fout, flse = torch.empty_like(fq), torch.empty((batch, HQ, tokens), device=device, dtype=torch.float32)
        replica_ms = timed(lambda: full_ops.forward_out(fq, fk, fv, fout, flse, empty, empty, 0, 1, SCALE, True),
                           args.steps, args.warmup)
        launches += args.steps
        prefill_replicas = {"workload": WORKLOAD + ", one whole batch per GPU (weak scaling, no shared work)",
                            "value": world * step_flops / (replica_ms / args.steps * 1e-3) / 1e12, "unit": UNIT,
                            "ms_per_step": replica_ms / args.steps}
        del fq, fk, fv, fout, flse
    del whole
    torch.cuda.empty_cache()

    # ------------------------------------------------------------------ shorter sequences (N = 1 only)
    # 2048-token batches run the persistent schedule of the prefill kernel; the headline runs one CTA per unit.
    prefill_shapes = None
    if world == 1:
        prefill_shapes = []
        full_ops = cuda_runtime.ops_for(library, "prefill")
        for sbatch, stokens in ((4, 2048), (1, 2048)):
            generator = torch.Generator(device=device).manual_seed(PREFILL["seed"] + stokens + sbatch)
            count = max(2, int(300e6 // (sbatch * stokens * HQ * DIM * 2 * 2.6)))  # rotate through more than L2 holds
            shape_sets = []
            for _ in range(count):
                sq = torch.randn((sbatch, stokens, HQ, DIM), generator=generator, device=device, dtype=torch.bfloat16)
                sk, sv = (torch.randn((sbatch, stokens, HKV, DIM), generator=generator, device=device,
                                      dtype=torch.bfloat16) for _ in range(2))
                shape_sets.append((sq, sk, sv, torch.empty_like(sq),
                                   torch.empty((sbatch, HQ, stokens), device=device, dtype=torch.float32)))
            shape_graphs = [graph_of(lambda t=t: full_ops.forward_out(t[0], t[1], t[2], t[3], t[4], empty, empty, 0, 1,
                                                                      SCALE, True)) for t in shape_sets]
            shape_turn = [0]

            def shape_step():
                shape_graphs[shape_turn[0] % count].replay()
                shape_turn[0] += 1

            shape_ms = timed(shape_step, max(args.steps, 20), max(args.warmup, 3)) / max(args.steps, 20)
            launches += max(args.steps, 20)
            tflops = prefill_flops(sbatch, stokens) / (shape_ms * 1e-3) / 1e12
            prefill_shapes.append({"workload": f"causal GQA prefill B{sbatch} S{stokens} Hq{HQ} Hkv{HKV} D{DIM}, graph replay over "
                                               f"{count} rotating buffer sets", "us_per_step": shape_ms * 1e3,
                                   "tflops": tflops, "frac_of_burst": tflops / peaks["bf16"]})
            del shape_graphs, shape_sets
            torch.cuda.empty_cache()

    # ------------------------------------------------------------------ decode
    def verify_sharded(driver, cache, dq, dkn, dvn, old, dout, dlse, shard_start, route):
        """One more step of a sharded route, outside any timed region, compared (a) bit for bit with the
        standalone combine of every rank's partial of the same shard (all-gathered), and (b) with the CPU oracle
        on two KV-head groups whose cache rows are gathered from all ranks."""
        kc, vc = cache
        cbatch, rows = dq.size(0), dq.size(0) * HQ
        dout.fill_(float("nan"))
        dlse.fill_(float("nan"))
        driver.step(dq, kc, vc, dkn, dvn, old, dout, dlse)
        packed = torch.empty(rows * (DIM + 1), device=device, dtype=torch.float32)
        part_o, part_lse = packed[:rows * DIM].view(rows, DIM), packed[rows * DIM:]
        spec = decode_ops.workspace_spec(dq, kc, old, 0, 1, True)
        scratch = [torch.empty(n, device=device, dtype=torch.float32) for n in spec[1:3]]
        decode_ops.partial_out(dq, kc, vc, dkn, dvn, old, part_o, part_lse, *scratch, 0, 1, True, shard_start)
        gathered = torch.empty((world, packed.numel()), device=device, dtype=torch.float32)
        dist.all_gather_into_tensor(gathered, packed)
        ref_o, ref_lse = torch.empty_like(dout), torch.empty_like(dlse)
        decode_ops.combine_partials(gathered[:, :rows * DIM].unflatten(1, (rows, DIM)), gathered[:, rows * DIM:], ref_o,
                                    ref_lse)
        torch.cuda.synchronize(device)

        def bits():
            assert torch.equal(dout.view(torch.int16), ref_o.view(torch.int16)), "O differs from the standalone combine"
            assert torch.equal(dlse.view(torch.int32), ref_lse.view(torch.int32)), "LSE differs from the standalone combine"
            return True

        def against_oracle():
            worst = [0.0, 0.0]
            for g in (0, 5):
                full = []
                for cache_part in (kc, vc):
                    mine = cache_part[:, :, g:g + 1].contiguous()
                    everyone = torch.empty((world, *mine.shape), device=device, dtype=mine.dtype)
                    dist.all_gather_into_tensor(everyone, mine)
                    full.append(everyone.permute(1, 0, 2, 3, 4).flatten(1, 2).cpu())  # [B, capacity, 1, 128]
                heads = slice(g * 4, (g + 1) * 4)
                want_o, want_lse, _, _ = oracle.decode_step(dq[:, :, heads].cpu(), full[0], full[1], dkn[:, :, g:g + 1].cpu(),
                                                            dvn[:, :, g:g + 1].cpu(), old.cpu())
                errors = oracle.check_outputs(dout[:, :, heads].cpu(), dlse[:, heads].cpu(), want_o, want_lse)
                worst = [max(a, b) for a, b in zip(worst, errors)]
            return worst

        bit_equal = checked(f"sharded decode ({route} route) vs standalone combine", bits) is not None
        worst = checked(f"sharded decode ({route} route) vs CPU oracle", against_oracle) or [float("inf")] * 2
        worst = [max_over_ranks(x) for x in worst]
        bit_equal = max_over_ranks(0.0 if bit_equal else 1.0) == 0.0
        ok = bit_equal and all(x != float("inf") for x in worst)
        return {"checked": ok, "bitwise_equal_to_standalone_combine": bit_equal,
                "against": "tc_combine_partials of the all-gathered per-rank partials (bits); CPU oracle on KV-head "
                           "groups 0 and 5 with cache rows gathered from all ranks",
                "o_max_abs": worst[0] if ok else None, "lse_rel": worst[1] if ok else None}

    def decode_case(case, sets, graph_steps, sharded):
        nonlocal launches
        cbatch, capacity, valid = case["batch"], case["capacity"], case["valid"]
        shard_start, shard_len = sharding.kv_sequence_shard(rank, world, capacity) if sharded else (0, capacity)
        generator = torch.Generator(device=device).manual_seed(case["seed"] + rank)
        caches = []
        for _ in range(sets):  # rotating cache sets: together larger than L2, so no step re-reads cached rows
            caches.append(tuple(torch.randn((cbatch, shard_len, HKV, DIM), generator=generator, device=device,
                                            dtype=torch.bfloat16) for _ in range(2)))
        # The query and the new rows are the same on every rank (a sharded step replicates them); only the cache
        # shards differ from rank to rank.
        shared_draws = torch.Generator(device=device).manual_seed(case["seed"] + 7919)
        dq = torch.randn((cbatch, 1, HQ, DIM), generator=shared_draws, device=device, dtype=torch.bfloat16)
        dkn, dvn = (torch.randn((cbatch, 1, HKV, DIM), generator=shared_draws, device=device, dtype=torch.bfloat16)
                    for _ in range(2))
        old = torch.full((cbatch,), valid, dtype=torch.int32, device=device)
        dout = torch.empty_like(dq)
        dlse = torch.empty((cbatch, HQ, 1), device=device, dtype=torch.float32)
        driver = None
        if sharded:
            driver = sharding.ShardedDecode(decode_ops, rank, world, cbatch, capacity, device, exchange=sharded)
            counter = [0]

            def step():
                kc, vc = caches[counter[0] % sets]
                counter[0] += 1
                driver.step(dq, kc, vc, dkn, dvn, old, dout, dlse)

            per_launch = 1 if sharded == "peer" else 2
            splits = None
        else:
            spec = decode_ops.workspace_spec(dq, caches[0][0], old, 0, 1, True)
            workspace = [torch.empty(n, device=device, dtype=torch.float32) for n in spec[1:3]]
            counter = [0]
            bound = [decode_ops.bind_forward_out(dq, kc, vc, dkn, dvn, old, dout, dlse, *workspace, 0, 1, True)
                     for kc, vc in caches]  # a serving loop validates its buffers once, then only launches

            def step():
                bound[counter[0] % sets]()
                counter[0] += 1

            per_launch = 1
            splits = spec[0]
        step()
        torch.cuda.synchronize(device)
        eager_ms = timed(step, graph_steps * 4, 3) / (graph_steps * 4)
        launches += graph_steps * 4 * per_launch
        checked_call_ms = None
        if not sharded:
            # The same steps through the reference-signature call, which validates its tensors every time.
            def checked_step():
                kc, vc = caches[counter[0] % sets]
                counter[0] += 1
                decode_ops.forward_out(dq, kc, vc, dkn, dvn, old, dout, dlse, *workspace, 0, 1, True)

            checked_call_ms = timed(checked_step, graph_steps * 4, 3) / (graph_steps * 4)
            launches += graph_steps * 4
        graph_ms = None
        try:
            # The kernel is a few microseconds long, so host launch cost hides it; replaying a captured
            # graph of `graph_steps` consecutive steps (kernel, all-gather and merge when sharded) shows
            # the device-side rate.
            stream = torch.cuda.Stream(device)
            with torch.cuda.stream(stream):
                step()
                stream.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    for _ in range(graph_steps):
                        step()
            replays = 10
            graph_ms = timed(graph.replay, replays, 3) / (replays * graph_steps)
            launches += replays * graph_steps * per_launch
        except Exception as error:  # graph capture of the collective is optional
            if not sharded:
                raise
            print(f"graph capture of the sharded step unavailable: {error}", file=sys.stderr)
            torch.cuda.synchronize(device)
        overlapped_ms = None
        if not sharded:
            # The same chain with the cache-stable promise: consecutive steps work on different cache sets (as the
            # layers of a model do), so each step may fetch its cache while its predecessor is still finishing.
            stable = [decode_ops.bind_forward_out(dq, kc, vc, dkn, dvn, old, dout, dlse, *workspace, 0, 1, True,
                                                  cache_stable=True) for kc, vc in caches]

            def stable_chain():
                for index in range(graph_steps):
                    stable[index % sets]()

            graph_stable = graph_of(stable_chain)
            overlapped_ms = timed(graph_stable.replay, 10, 3) / (10 * graph_steps)
            launches += 10 * graph_steps
        attended = min(max(valid + 1 - shard_start, 0), shard_len)
        rank_bytes = decode_bytes(cbatch, attended)
        best_ms = min(x for x in (eager_ms, graph_ms) if x is not None)
        gbs = rank_bytes / (best_ms * 1e-3) / 1e9
        result = {"batch": cbatch, "capacity": capacity, "attended_rows": valid + 1, "splits": splits,
                  "us_per_step_eager": eager_ms * 1e3, "us_per_step_graph": None if graph_ms is None else graph_ms * 1e3,
                  "entry": ("sharding.ShardedDecode.step" if sharded else
                            "us_per_step_eager: DecodeOps.bind_forward_out (buffers validated once, then launches "
                            "only; not in the reference); us_per_step_eager_forward_out: DecodeOps.forward_out, the "
                            "reference-signature call; us_per_step_graph: graph replay of the same launches, which "
                            "holds no host call path at all. hbm_gbs_per_gpu uses the fastest of them"),
                  "us_per_step_eager_forward_out": None if checked_call_ms is None else checked_call_ms * 1e3,
                  "hbm_gbs_per_gpu": gbs, "bytes_per_step_per_gpu": rank_bytes,
                  "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s",
                               "frac": gbs / peaks["hbm"],
                               "traffic": None if sharded else NCU_TRAFFIC_BYTES["decode_c4" if cbatch == 1 else "decode_c5"],
                               "peak_source": peaks["source"]},
                  "cache_sets": sets}
        if overlapped_ms is not None:
            overlapped_gbs = rank_bytes / (overlapped_ms * 1e-3) / 1e9
            result["us_per_step_graph_cache_stable"] = overlapped_ms * 1e3
            result["roofline_cache_stable"] = {
                "bound": "hbm", "achieved": overlapped_gbs, "peak": peaks["hbm"], "unit": "GB/s",
                "frac": overlapped_gbs / peaks["hbm"], "peak_source": peaks["source"],
                "what": "steady state of a chain of steps on different caches launched with TC_DECODE_CACHE_STABLE: a step "
                        "streams its cache (ring + L2 prefetch) while the step before it finishes; graph replay"}
        if driver is not None:
            result["check"] = verify_sharded(driver, caches[0], dq, dkn, dvn, old, dout, dlse, shard_start, sharded)
            torch.cuda.synchronize(device)
            driver.close()
        del caches
        torch.cuda.empty_cache()
        return result

    decode = {"c4": decode_case(DECODE_C4, sets=8, graph_steps=16, sharded=None)}
    decode["c4"]["workload"] = "config4 B1 capacity 32768, 8192 valid + 1 appended, replicas at N>1"
    if world > 1 and DECODE_C5["capacity"] % world == 0:
        nccl_note = ("decode kernel, one NCCL all-gather of packed partial O/LSE, LSE combine kernel: three launches per "
                     "step")
        try:
            decode["c5"] = decode_case(DECODE_C5, sets=2, graph_steps=4, sharded="peer")
            decode["c5"]["workload"] = (f"config5 B4 32768 rows attended, KV sequence sharded over {world} GPUs, one "
                                        "launch per step: partial O/LSE cross NVLink as peer stores inside the decode "
                                        "kernel, which also merges them")
        except RuntimeError as error:  # agreed on by all ranks (see sharding.PeerBlocks)
            print(f"in-launch exchange unavailable, using the library route: {error}", file=sys.stderr)
            decode["c5"] = None
        decode["c5_nccl"] = decode_case(DECODE_C5, sets=2, graph_steps=4, sharded="nccl")
        decode["c5_nccl"]["workload"] = f"config5 B4, KV sequence sharded over {world} GPUs, library route: {nccl_note}"
        if decode["c5"] is None:
            decode["c5"] = decode.pop("c5_nccl")
    else:
        decode["c5"] = decode_case(DECODE_C5, sets=2, graph_steps=4, sharded=None)
        decode["c5"]["workload"] = "config5 B4 32768 rows attended (new row lands at index 32767), one GPU"

    # ------------------------------------------------------------------ the step before decode (replicas at N > 1)
    def project_case(tokens, hidden=2560, sets=8, graph_steps=16):
        nonlocal launches
        ops = cuda_runtime.ops_for(library, "project")
        rows = (HQ + 2 * HKV) * DIM
        generator = torch.Generator(device=device).manual_seed(7 + rank)
        weights = [(torch.randn((rows, hidden), generator=generator, device=device) / hidden ** 0.5).to(torch.bfloat16)
                   for _ in range(sets)]  # rotating weight sets, together larger than L2
        x = torch.randn((tokens, hidden), generator=generator, device=device).to(torch.bfloat16)
        norm = [torch.ones(DIM, device=device, dtype=torch.bfloat16) for _ in range(2)]
        angles = torch.rand((32768, DIM // 2), generator=generator, device=device)
        cos, sin = angles.cos(), angles.sin()
        positions = torch.full((tokens,), 8192, dtype=torch.int32, device=device)
        outs = [torch.empty((tokens, 1, heads, DIM), device=device, dtype=torch.bfloat16) for heads in (HQ, HKV, HKV)]
        counter = [0]
        replays = 10
        moved = rows * hidden * 2 + tokens * hidden * 2 + tokens * (HQ + 2 * HKV) * DIM * 2

        def chain_ms(release_early):
            nonlocal launches

            def step():
                ops.forward_out(x, weights[counter[0] % sets], positions, *outs, q_norm_weight=norm[0],
                                k_norm_weight=norm[1], rope_cos=cos, rope_sin=sin, release_early=release_early)
                counter[0] += 1

            step()
            torch.cuda.synchronize(device)
            stream = torch.cuda.Stream(device)
            with torch.cuda.stream(stream):
                step()
                stream.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    for _ in range(graph_steps):
                        step()
            launches += replays * graph_steps
            return timed(graph.replay, replays, 3) / (replays * graph_steps)

        def roofline(ms):
            gbs = moved / (ms * 1e-3) / 1e9
            return {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s", "frac": gbs / peaks["hbm"],
                    "traffic": NCU_TRAFFIC_BYTES["project"] if (tokens, hidden) == (4, 2560) else None,
                    "peak_source": peaks["source"]}

        ms, early_ms = chain_ms(False), chain_ms(True)
        return {"workload": f"fused QKV projection + head RMS norm + RoPE, {tokens} token(s), hidden {hidden}, "
                            f"{HQ}+{HKV}+{HKV} heads (Qwen3-4B shapes), weights streamed from HBM",
                "us_per_step_graph": ms * 1e3, "bytes_per_step": moved, "roofline": roofline(ms),
                "us_per_step_graph_release_early": early_ms * 1e3,
                "roofline_release_early": dict(roofline(early_ms), what="the same chain launched with "
                                               "TC_PROJECT_RELEASE_EARLY: a launch's weight stream starts while the "
                                               "launch two places before it is still running")}

    try:
        project = project_case(tokens=4)
    except RuntimeError as error:  # an extra beside the headline numbers: never lose the line over it
        print(f"projection step not measured: {error}", file=sys.stderr)
        project = {"unavailable": str(error)}

    # ------------------------------------------------------------------ projection -> decode, as a layer runs them
    def layer_chain_case(sets=8, graph_steps=16):
        """One token's projection followed by the config-4 decode step on that layer's cache, `graph_steps`
        layers back to back in a captured graph; once with the plain decode entry, once with the cache-stable
        promise, under which the decode kernel streams K/V while the projection finishes, and once with the
        projection's early release on top."""
        nonlocal launches
        project_ops = cuda_runtime.ops_for(library, "project")
        hidden, rows = 2560, (HQ + 2 * HKV) * DIM
        capacity, valid = DECODE_C4["capacity"], DECODE_C4["valid"]
        generator = torch.Generator(device=device).manual_seed(11 + rank)
        weights = [(torch.randn((rows, hidden), generator=generator, device=device) / hidden ** 0.5).to(torch.bfloat16)
                   for _ in range(sets)]
        caches = [tuple(torch.randn((1, capacity, HKV, DIM), generator=generator, device=device, dtype=torch.bfloat16)
                        for _ in range(2)) for _ in range(sets)]
        x = torch.randn((1, hidden), generator=generator, device=device).to(torch.bfloat16)
        angles = torch.rand((capacity, DIM // 2), generator=generator, device=device)
        cos, sin = angles.cos(), angles.sin()
        old = torch.full((1,), valid, dtype=torch.int32, device=device)
        q, knew, vnew = (torch.empty((1, 1, heads, DIM), device=device, dtype=torch.bfloat16) for heads in (HQ, HKV, HKV))
        out, lse = torch.empty_like(q), torch.empty((1, HQ, 1), device=device, dtype=torch.float32)
        spec = decode_ops.workspace_spec(q, caches[0][0], old, 0, 1, True)
        workspace = [torch.empty(n, device=device, dtype=torch.float32) for n in spec[1:3]]
        result = {"workload": "per layer: fused QKV projection (1 token, hidden 2560) then config4 decode step on that "
                              f"layer's cache; {sets} rotating weight and cache sets (larger than L2), {graph_steps} "
                              "layers per captured graph"}
        # Third arm: the projection also releases its follower early (TC_PROJECT_RELEASE_EARLY), so the decode step of
        # a layer streams its cache beside the decode step of the layer before it as well; in a model that step works
        # on another layer's cache, so the cache-stable promise holds for both predecessors (here: another cache set).
        for key, promise, early in (("us_per_layer", False, False), ("us_per_layer_cache_stable", True, False),
                                    ("us_per_layer_cache_stable_release_early", True, True)):
            steps = [decode_ops.bind_forward_out(q, kc, vc, knew, vnew, old, out, lse, *workspace, 0, 1, True,
                                                 cache_stable=promise) for kc, vc in caches]

            def chain():
                for layer in range(graph_steps):
                    project_ops.forward_out(x, weights[layer % sets], old, q, knew, vnew, rope_cos=cos, rope_sin=sin,
                                            release_early=early)
                    steps[layer % sets]()

            chain()
            torch.cuda.synchronize(device)
            stream = torch.cuda.Stream(device)
            with torch.cuda.stream(stream):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    chain()
            replays = 10
            result[key] = timed(graph.replay, replays, 3) / (replays * graph_steps) * 1e3
            launches += replays * graph_steps * 2
        moved = rows * hidden * 2 + decode_bytes(1, valid + 1)
        result["bytes_per_layer"] = moved
        result["hbm_gbs_cache_stable"] = moved / (result["us_per_layer_cache_stable"] * 1e-6) / 1e9
        result["hbm_gbs_cache_stable_release_early"] = moved / (result["us_per_layer_cache_stable_release_early"] * 1e-6) / 1e9
        return result

    try:
        layer_chain = layer_chain_case()
    except RuntimeError as error:
        print(f"projection -> decode chain not measured: {error}", file=sys.stderr)
        layer_chain = {"unavailable": str(error)}

    status = library.device_status(device.index)
    if status != 0:
        raise RuntimeError(f"a kernel reported an expired wait (status {status}); results are invalid")
    if world > 1:
        for key in ("c5", "c5_nccl"):
            if decode.get(key) and "check" in decode[key]:
                checks[key] = decode[key]["check"]
        failed = max_over_ranks(float(len(check_failures)))
        if failed:
            if rank == 0:
                print("result checks failed; no benchmark line is printed", file=sys.stderr, flush=True)
            dist.barrier()
            dist.destroy_process_group()
            raise SystemExit(1)

    # ------------------------------------------------------------------ CPU baseline (rank 0, N = 1)
    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        cpu_value, threads, description, _ = cpu_attention_sample(torch, oracle, seconds_hint=12.0, kv_groups=HKV)
        cpu_baseline = {"value": cpu_value, "unit": UNIT, "cores": threads, "kind": "port", "sample": description}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": bench_config(world), "prefill": {"ctas_per_query_tile": ctas_per_query_tile, "buffer_sets": sets},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["bf16"], "frac_of_sustained": achieved / peaks["bf16_sustained"],
                         "traffic": NCU_TRAFFIC_BYTES["prefill_c2"] if world == 1 else None,
                         "peak_source": peaks["source"] + " burst", "per": "GPU"},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                    "ms_per_step": e2e_ms / args.steps, "bytes": "all ranks together"},
            "clocks": clocks, "gpu_launches": launches, "decode": decode, "project": project,
            "layer_chain": layer_chain,
        }
        if prefill_replicas:
            line["prefill_replicas"] = prefill_replicas
        if prefill_shapes is not None:
            line["prefill_shapes"] = prefill_shapes
        if checks:
            line["checks"] = checks
        if cpu_baseline:
            line["cpu_baseline"] = cpu_baseline
        json_out.write(json.dumps(line) + "\n")
        json_out.flush()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs {args.gpus} ranks (torch.distributed.run), found WORLD_SIZE={world}")
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()

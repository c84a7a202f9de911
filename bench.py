"""Benchmark of the B200 attention hot path: causal GQA prefill (headline) and split-KV decode.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

For N > 1 launch with ``python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N``.
Rank 0 prints ONE JSON line.

Headline workload (``config.workload``): BASELINE config 2, causal prefill, BF16, batch 1, 8192
tokens, 32 query / 8 KV heads, D = 128, N(0,1) inputs from seed 1 (synthetic stand-ins for the
reference's saved Qwen3 projections). A step is one forward over that batch.

* ``value``      TFLOP/s (4*B*Hq*S^2*D/2 per step) with inputs resident in HBM, all ranks together.
                 At N > 1 every rank runs its own batch of the same shape (the units are (batch, KV-head
                 group) pairs, eight per rank, no collective): weak scaling.
* ``e2e``        the same metric through the operator API with HOST buffers: every step copies its
                 Q/K/V from pinned host memory and reads O and LSE back; copies and kernels of
                 neighbouring steps overlap on three streams.
* ``roofline``   the prefill kernel against the measured dense BF16 peak.
* ``decode``     split-KV decode with fused append: config 4 (batch 1, 8192 of 32768 rows valid) and
                 config 5 (batch 4, 32768 rows attended; KV sequence sharded over the ranks when N > 1 and
                 merged inside the decode launch over NVLink, with the all-gather + combine route beside
                 it as ``c5_nccl``), as HBM GB/s with their own roofline.
* ``project``    the step before decode (fused QKV projection + head RMS norm + RoPE, 4 tokens, Qwen3-4B
                 shapes) as HBM GB/s of streamed weights.
* ``layer_chain`` projection then config-4 decode as a layer runs them, microseconds per layer, with the plain
                 decode entry and with the cache-stable promise (K/V streamed while the projection finishes).
* ``prefill_sharded`` (N > 1) config 2 itself split by KV-head group over the ranks (strong scaling).
* ``cpu_baseline`` the CPU oracle (the reference's only CPU attention, ``bench_exchange.py:54-60``)
                 timed on this host on a bounded sample.

``--impl reference`` times that CPU attention alone, on rank 0, with all host threads.
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


def prefill_flops(batch, tokens, heads=HQ):
    return 4.0 * batch * heads * tokens * tokens * DIM / 2.0


def decode_bytes(batch, attended, kv_heads=HKV):
    """Algorithmic HBM bytes of one decode step: K and V rows attended, Q in, O out, LSE, new rows in + out."""
    q_heads = kv_heads * 4
    return (2 * batch * attended * kv_heads * DIM * 2 + 2 * batch * q_heads * DIM * 2 + batch * q_heads * 4
            + 4 * batch * kv_heads * DIM * 2)


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
def cpu_attention_sample(torch, oracle, seconds_hint=10.0, steps=None, warmup=0):
    """Time the CPU oracle on one KV-head group (4 query heads) of the headline workload.

    Returns (TFLOP/s, threads, description, seconds per pass). The sample is 1/8 of a step's FLOPs;
    throughput is per FLOP, so no scaling is applied.
    """
    torch.set_num_threads(os.cpu_count() or 1)
    tokens = PREFILL["tokens"]
    q, k, v = oracle.seeded_normal(PREFILL["seed"], (1, tokens, 4, DIM), (1, tokens, 1, DIM), (1, tokens, 1, DIM))
    flops = prefill_flops(1, tokens, heads=4)
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
    description = (f"one KV-head group (4 of 32 query heads, all {tokens} rows) of the config-2 prefill, "
                   f"{len(times)} passes, median")
    return flops / best / 1e12, torch.get_num_threads(), description, best


def run_reference(args, rank):
    if rank != 0:
        return
    import torch
    from oracle import attention as oracle

    value, threads, description, seconds = cpu_attention_sample(torch, oracle, steps=max(1, args.steps),
                                                                warmup=args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "config2 causal GQA prefill B1 S8192 Hq32 Hkv8 D128 seed1 (CPU sample)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": description},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------- GPU arm
def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from oracle import attention as oracle  # CPU baseline leg only
    from tilecadence_b200 import cuda_runtime, sharding

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
    prefill_ops = cuda_runtime.ops_for(library, "prefill")
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

    # ------------------------------------------------------------------ prefill, resident inputs
    batch, tokens = PREFILL["batch"], PREFILL["tokens"]
    host = oracle.seeded_normal(PREFILL["seed"] + 1000 * rank, (batch, tokens, HQ, DIM), (batch, tokens, HKV, DIM),
                                (batch, tokens, HKV, DIM))
    host = [tensor.pin_memory() for tensor in host]
    q, k, v = (tensor.to(device) for tensor in host)
    out = torch.empty_like(q)
    lse = torch.empty((batch, HQ, tokens), device=device, dtype=torch.float32)
    empty = torch.empty(0, device=device, dtype=torch.float32)

    def prefill_step():
        prefill_ops.forward_out(q, k, v, out, lse, empty, empty, 0, 1, SCALE, True)

    uuid = str(torch.cuda.get_device_properties(device).uuid)
    uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
    sampler = ClockSampler(uuid)  # stays open over the resident and the host-buffer timed regions
    sampler.__enter__()
    prefill_ms = timed(prefill_step, args.steps, args.warmup)
    launches += args.steps
    ms_per_step = prefill_ms / args.steps
    step_flops = prefill_flops(batch, tokens)
    value = world * step_flops / (ms_per_step * 1e-3) / 1e12
    achieved = step_flops / (ms_per_step * 1e-3) / 1e12

    # ------------------------------------------------------------------ prefill, host buffers (e2e)
    host_out = [torch.empty(out.shape, dtype=out.dtype).pin_memory() for _ in range(2)]
    host_lse = [torch.empty(lse.shape, dtype=lse.dtype).pin_memory() for _ in range(2)]
    slots = [dict(q=torch.empty_like(q), k=torch.empty_like(k), v=torch.empty_like(v), out=torch.empty_like(out),
                  lse=torch.empty_like(lse)) for _ in range(2)]
    copy_in, compute, copy_out = (torch.cuda.Stream(device) for _ in range(3))

    def e2e_run(steps):
        loaded = [None, None]
        computed = [None, None]
        drained = [None, None]
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(copy_in)
        for index in range(steps):
            slot = slots[index % 2]
            with torch.cuda.stream(copy_in):
                if computed[index % 2] is not None:
                    copy_in.wait_event(computed[index % 2])  # the kernel that read this slot is done
                for name, source in zip("qkv", host):
                    slot[name].copy_(source, non_blocking=True)
                loaded[index % 2] = torch.cuda.Event()
                loaded[index % 2].record(copy_in)
            with torch.cuda.stream(compute):
                compute.wait_event(loaded[index % 2])
                if drained[index % 2] is not None:
                    compute.wait_event(drained[index % 2])  # the previous result left this slot
                prefill_ops.forward_out(slot["q"], slot["k"], slot["v"], slot["out"], slot["lse"], empty, empty, 0, 1,
                                        SCALE, True)
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
    e2e_value = world * step_flops / (e2e_ms / args.steps * 1e-3) / 1e12
    h2d_bytes = sum(t.numel() * t.element_size() for t in host)
    d2h_bytes = out.numel() * out.element_size() + lse.numel() * lse.element_size()
    del slots, host_out, host_lse

    # ------------------------------------------------------------------ prefill sharded by KV-head group (N > 1)
    prefill_sharded = None
    if world > 1 and HKV % world == 0:
        kv_slice, q_slice = sharding.kv_head_slice(rank, world, HKV)
        shared = oracle.seeded_normal(PREFILL["seed"], (batch, tokens, HQ, DIM), (batch, tokens, HKV, DIM),
                                      (batch, tokens, HKV, DIM))
        sq = shared[0][:, :, q_slice].contiguous().to(device)
        sk = shared[1][:, :, kv_slice].contiguous().to(device)
        sv = shared[2][:, :, kv_slice].contiguous().to(device)
        shard_ops = cuda_runtime.ops_for(library, "prefill", q_heads=HQ // world)
        sout, slse = torch.empty_like(sq), torch.empty((batch, HQ // world, tokens), device=device)
        # A shard of few heads cannot fill the GPU with one CTA per query tile: the key-split entry then
        # gives every tile to two CTAs (its own choice; one CTA per tile is the plain kernel).
        split_ws = torch.empty(shard_ops.key_split_workspace_bytes(sq), device=device, dtype=torch.uint8)
        key_splits = shard_ops.key_split_forward_out(sq, sk, sv, sout, slse, split_ws, 1, SCALE, 0)
        shard_ms = timed(lambda: shard_ops.key_split_forward_out(sq, sk, sv, sout, slse, split_ws, 1, SCALE, 0),
                         args.steps, args.warmup)
        launches += args.steps
        prefill_sharded = {"workload": "config2 split by KV-head group over the ranks (strong scaling, no collective)",
                           "value": step_flops / (shard_ms / args.steps * 1e-3) / 1e12, "unit": UNIT,
                           "ms_per_step": shard_ms / args.steps, "ctas_per_query_tile": key_splits}
        del sq, sk, sv, sout, slse, shared, split_ws
    del q, k, v, out, lse
    torch.cuda.empty_cache()

    # ------------------------------------------------------------------ decode
    def decode_case(case, sets, graph_steps, sharded):
        nonlocal launches
        cbatch, capacity, valid = case["batch"], case["capacity"], case["valid"]
        shard_start, shard_len = sharding.kv_sequence_shard(rank, world, capacity) if sharded else (0, capacity)
        generator = torch.Generator(device=device).manual_seed(case["seed"] + rank)
        caches = []
        for _ in range(sets):  # rotating cache sets: together larger than L2, so no step re-reads cached rows
            caches.append(tuple(torch.randn((cbatch, shard_len, HKV, DIM), generator=generator, device=device,
                                            dtype=torch.bfloat16) for _ in range(2)))
        dq = torch.randn((cbatch, 1, HQ, DIM), generator=generator, device=device, dtype=torch.bfloat16)
        dkn, dvn = (torch.randn((cbatch, 1, HKV, DIM), generator=generator, device=device, dtype=torch.bfloat16)
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
        attended = min(max(valid + 1 - shard_start, 0), shard_len)
        rank_bytes = decode_bytes(cbatch, attended)
        best_ms = min(x for x in (eager_ms, graph_ms) if x is not None)
        gbs = rank_bytes / (best_ms * 1e-3) / 1e9
        result = {"batch": cbatch, "capacity": capacity, "attended_rows": valid + 1, "splits": splits,
                  "us_per_step_eager": eager_ms * 1e3, "us_per_step_graph": None if graph_ms is None else graph_ms * 1e3,
                  "hbm_gbs_per_gpu": gbs, "bytes_per_step_per_gpu": rank_bytes,
                  "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s",
                               "frac": gbs / peaks["hbm"],
                               "traffic": None if sharded else NCU_TRAFFIC_BYTES["decode_c4" if cbatch == 1 else "decode_c5"],
                               "peak_source": peaks["source"]},
                  "cache_sets": sets}
        if driver is not None:
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

        def step():
            ops.forward_out(x, weights[counter[0] % sets], positions, *outs, q_norm_weight=norm[0],
                            k_norm_weight=norm[1], rope_cos=cos, rope_sin=sin)
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
        replays = 10
        ms = timed(graph.replay, replays, 3) / (replays * graph_steps)
        launches += replays * graph_steps
        moved = rows * hidden * 2 + tokens * hidden * 2 + tokens * (HQ + 2 * HKV) * DIM * 2
        gbs = moved / (ms * 1e-3) / 1e9
        return {"workload": f"fused QKV projection + head RMS norm + RoPE, {tokens} token(s), hidden {hidden}, "
                            f"{HQ}+{HKV}+{HKV} heads (Qwen3-4B shapes), weights streamed from HBM",
                "us_per_step_graph": ms * 1e3, "bytes_per_step": moved,
                "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s",
                             "frac": gbs / peaks["hbm"], "traffic": NCU_TRAFFIC_BYTES["project"] if (tokens, hidden) == (4, 2560) else None,
                             "peak_source": peaks["source"]}}

    try:
        project = project_case(tokens=4)
    except RuntimeError as error:  # an extra beside the headline numbers: never lose the line over it
        print(f"projection step not measured: {error}", file=sys.stderr)
        project = {"unavailable": str(error)}

    # ------------------------------------------------------------------ projection -> decode, as a layer runs them
    def layer_chain_case(sets=8, graph_steps=16):
        """One token's projection followed by the config-4 decode step on that layer's cache, `graph_steps`
        layers back to back in a captured graph; once with the plain decode entry and once with the
        cache-stable promise, under which the decode kernel streams K/V while the projection finishes."""
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
        for key, promise in (("us_per_layer", False), ("us_per_layer_cache_stable", True)):
            steps = [decode_ops.bind_forward_out(q, kc, vc, knew, vnew, old, out, lse, *workspace, 0, 1, True,
                                                 cache_stable=promise) for kc, vc in caches]

            def chain():
                for layer in range(graph_steps):
                    project_ops.forward_out(x, weights[layer % sets], old, q, knew, vnew, rope_cos=cos, rope_sin=sin)
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
        return result

    try:
        layer_chain = layer_chain_case()
    except RuntimeError as error:
        print(f"projection -> decode chain not measured: {error}", file=sys.stderr)
        layer_chain = {"unavailable": str(error)}

    status = library.device_status(device.index)
    if status != 0:
        raise RuntimeError(f"a kernel reported an expired wait (status {status}); results are invalid")

    # ------------------------------------------------------------------ CPU baseline (rank 0, N = 1)
    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        cpu_value, threads, description, _ = cpu_attention_sample(torch, oracle, seconds_hint=12.0)
        cpu_baseline = {"value": cpu_value, "unit": UNIT, "cores": threads, "kind": "port", "sample": description}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "config2 causal GQA prefill B1 S8192 Hq32 Hkv8 D128 seed1, one batch per GPU",
                       "l2": "inputs+outputs 161 MiB per step, larger than the 126 MB L2",
                       "decode_l2": "rotating cache sets larger than L2"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["bf16"], "frac_of_sustained": achieved / peaks["bf16_sustained"],
                         "traffic": NCU_TRAFFIC_BYTES["prefill_c2"], "peak_source": peaks["source"] + " burst"},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                    "ms_per_step": e2e_ms / args.steps},
            "clocks": clocks, "gpu_launches": launches, "decode": decode, "project": project,
            "layer_chain": layer_chain,
        }
        if prefill_sharded:
            line["prefill_sharded"] = prefill_sharded
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

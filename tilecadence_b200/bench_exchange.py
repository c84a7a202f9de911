"""Verify and time the four generated two-tile attention schedules on a B200.

The procedure is the one of ``tilecadence/bench_exchange.py`` (fp32 attention on the device tensors as
the yardstick :54-60, tolerances :63-66, arm-against-arm check :96-113, CUDA-graph timing :116-163,
driver :194-232); the code is this build's. For each arm the plan is solved, certified
(:func:`tilecadence_b200.exchange.verify`), emitted and compiled. ``retain`` must match the yardstick
(O: atol/rtol 0.003/0.01 for FP16, 0.02/0.02 for BF16; LSE: 5e-4/1e-4) on every buffer set; each
exchange arm must reproduce ``retain`` bit for bit. Timing replays a CUDA graph of ``LAUNCHES_PER_GRAPH``
launches, once always on the same buffer set and once walking over all ``--slots`` sets, and reports
the median per-launch time and the ratio to ``retain``. There is no stock-FlashAttention arm: this
build has one backend. ``<work>/result.json`` and ``<work>/build.json`` are written; ``--work`` must
not exist.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path
from statistics import median

from . import exchange, model
from .cuda_runtime import build_cuda, cuda_device
from .emit_exchange import RESOURCE_KEYS, emit

BASELINE_ARM = "retain"
EXCHANGE_ARMS = tuple(arm for arm in exchange.ARMS if arm != BASELINE_ARM)
LAUNCHES_PER_GRAPH = 16
GRAPH_REPLAYS = 32
TOKENS, HEAD_DIM = 64, 128
O_TOLERANCE = {"float16": (3e-3, 1e-2), "bfloat16": (2e-2, 2e-2)}  # (atol, rtol)
LSE_TOLERANCE = (5e-4, 1e-4)


class BufferSet:
    """Inputs and preallocated outputs of one launch: q, k, v, out [B,64,H,128] and lse [B,H,64]."""

    def __init__(self, torch, generator, batch, heads, dtype, device):
        dims = (batch, TOKENS, heads, HEAD_DIM)
        self.q, self.k, self.v = (torch.randn(dims, generator=generator, device=device, dtype=dtype) for _ in range(3))
        self.out = torch.empty(dims, device=device, dtype=dtype)
        self.lse = torch.empty((batch, heads, TOKENS), device=device, dtype=torch.float32)

    def yardstick(self, torch, causal):
        """fp32 attention of this set: O [B,64,H,128] and natural-log LSE [B,H,64]."""
        q, k, v = (tensor.float().permute(0, 2, 1, 3) for tensor in (self.q, self.k, self.v))  # B,H,S,D
        logits = torch.matmul(q, k.transpose(2, 3)) / HEAD_DIM ** 0.5
        if causal:
            hidden = torch.ones((TOKENS, TOKENS), dtype=torch.bool, device=logits.device).triu(1)
            logits = logits.masked_fill(hidden, float("-inf"))
        lse = torch.logsumexp(logits, dim=-1)
        return torch.matmul(torch.softmax(logits, dim=-1), v).permute(0, 2, 1, 3), lse


class ArmRunner:
    """One compiled arm: ``launch(buffers)`` enqueues it and returns the buffers' (out, lse)."""

    def __init__(self, name, ops, causal, plan):
        self.name, self.ops, self.causal = name, ops, causal
        self.summary = {"status": plan["status"], "source_steps": plan["finish_step"], "objective": plan["objective"]}

    def launch(self, buffers: BufferSet):
        self.ops.forward_out(buffers.q, buffers.k, buffers.v, buffers.out, buffers.lse, None, self.causal, True, False)
        return buffers.out, buffers.lse


def build_arm(name, work: Path, device, causal, seconds):
    problem = exchange.build_problem(name)
    plan = model.solve(problem, max_time_seconds=seconds)
    exchange.verify(problem.provenance[exchange.PROVENANCE_KEY], plan)
    directory = work / name / "emitted"
    emit(problem, plan, directory)
    ops, identity = build_cuda(directory, None, device)
    return ArmRunner(name, ops, causal, plan), identity


def check_arms(torch, runners, buffer_sets, causal, dtype_name):
    """``retain`` against the fp32 yardstick, then every other arm against ``retain``, on every set."""
    o_atol, o_rtol = O_TOLERANCE[dtype_name]
    baseline = runners[BASELINE_ARM]
    for buffers in buffer_sets:
        want_o, want_lse = buffers.yardstick(torch, causal)
        got_o, got_lse = baseline.launch(buffers)
        torch.testing.assert_close(got_o.float(), want_o, atol=o_atol, rtol=o_rtol)
        torch.testing.assert_close(got_lse, want_lse, atol=LSE_TOLERANCE[0], rtol=LSE_TOLERANCE[1])
        kept_o, kept_lse = got_o.clone(), got_lse.clone()
        for name in EXCHANGE_ARMS:
            other_o, other_lse = runners[name].launch(buffers)
            same = (torch.equal(other_o.view(torch.int16), kept_o.view(torch.int16))
                    and torch.equal(other_lse.view(torch.int32), kept_lse.view(torch.int32)))
            if not same:
                raise RuntimeError(f"{name} differs bitwise from the retain schedule")


def graph_time_us(torch, runner: ArmRunner, buffer_sets, walk: bool) -> float:
    """Median per-launch microseconds over ``GRAPH_REPLAYS`` replays of a captured launch sequence."""
    sequence = [buffer_sets[index % len(buffer_sets)] if walk else buffer_sets[0] for index in range(LAUNCHES_PER_GRAPH)]
    runner.launch(buffer_sets[0])  # anything lazy happens outside the capture
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side), torch.cuda.graph(graph, stream=side):
        for buffers in sequence:
            runner.launch(buffers)
    per_launch = []
    for _ in range(GRAPH_REPLAYS):
        begin, finish = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        graph.replay()
        finish.record()
        finish.synchronize()
        per_launch.append(begin.elapsed_time(finish) * 1e3 / LAUNCHES_PER_GRAPH)
    return median(per_launch)


def run(args):
    import torch

    args.work.mkdir(parents=True, exist_ok=False)
    device, _ = cuda_device(args.device)
    dtype = {"float16": torch.float16, "bfloat16": torch.bfloat16}[args.dtype]
    with torch.cuda.device(device), torch.inference_mode():
        runners, identities = {}, {}
        for name in exchange.ARMS:
            runners[name], identities[name] = build_arm(name, args.work, device, args.causal, args.seconds)
        generator = torch.Generator(device=device).manual_seed(args.seed)
        buffer_sets = [BufferSet(torch, generator, args.batch, args.heads, dtype, device) for _ in range(args.slots)]
        last = runners[exchange.ARMS[-1]].ops
        resources = dict(zip(RESOURCE_KEYS, last.resources(buffer_sets[0].q, args.causal), strict=True))
        if resources["theoretical_active_ctas_per_sm"] < 1 or resources["diagnostic_guard"]:
            raise RuntimeError(f"Generated kernel cannot be used for benchmarking: {resources}")
        check_arms(torch, runners, buffer_sets, args.causal, args.dtype)
        if any(runner.ops.library.device_status(device.index) != 0 for runner in runners.values()):
            raise RuntimeError("A kernel reported an expired wait")
        report = {name: dict(runner.summary) for name, runner in runners.items()}
        if not args.verify_only:
            for name, runner in runners.items():
                report[name]["repeated_us"] = graph_time_us(torch, runner, buffer_sets, walk=False)
                report[name]["rotating_us"] = graph_time_us(torch, runner, buffer_sets, walk=True)
            for name in EXCHANGE_ARMS:
                for mode in ("repeated", "rotating"):
                    report[name][f"{mode}_speedup_vs_retain"] = report[BASELINE_ARM][f"{mode}_us"] / report[name][f"{mode}_us"]
    record = {"dtype": args.dtype, "causal": args.causal, "batch": args.batch, "heads": args.heads,
              "slots": args.slots, "verified": True, "resources": resources, "arms": report}
    (args.work / "result.json").write_text(json.dumps(record, indent=2) + "\n")
    (args.work / "build.json").write_text(json.dumps(identities, indent=2) + "\n")
    print(json.dumps(record), flush=True)
    return record


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--work", required=True, type=Path)
    parser.add_argument("--flash-attention-root", type=Path, help="ignored: no FlashAttention checkout is needed")
    parser.add_argument("--device", default="cuda:0")
    parser.add_argument("--dtype", default="float16", choices=sorted(O_TOLERANCE))
    parser.add_argument("--causal", action="store_true")
    parser.add_argument("--batch", default=1, type=int)
    parser.add_argument("--heads", default=192, type=int)
    parser.add_argument("--slots", default=16, type=int)
    parser.add_argument("--seed", default=0, type=int)
    parser.add_argument("--seconds", default=2, type=float)
    parser.add_argument("--verify-only", action="store_true")
    args = parser.parse_args(argv)
    if min(args.batch, args.heads, args.slots) < 1:
        parser.error("batch, heads and slots must be positive")
    run(args)


if __name__ == "__main__":
    main()

"""Verify and time the emitted prefill or decode operator on a B200: the two-arm harness.

Command line, checks and output files follow ``tilecadence/bench_operator.py`` (verification of
prefill :29-43 and decode :46-78, guarded timing :81-95, driver :98-152) so that rows can be read
side by side with the reference's: ``--work`` is created fresh and receives ``rows.jsonl`` (one JSON
row per batch x length, also printed) and ``build.json`` (the build identity). ``--source`` names a
directory emitted earlier by :mod:`tilecadence_b200.operator`; without it the phase is emitted into
``<work>/source`` first. ``--flash-attention-root`` is accepted and ignored.

A row is produced in three stages. *Set-up*: seeded N(0,1) BF16 tensors, both arms (mapping 0 = the
kernel with a dedicated staging area, mapping 1 = the planner-placed handoff) run once. *Verification*:
the arms must agree bit for bit in O (16-bit words) and LSE (32-bit words) and be finite; for decode,
two consecutive steps are run per arm and the cache must hold the untouched history and both appended
rows bit for bit. *Timing* (unless ``--verify-only``): ``--rounds`` alternating pairs, each call
bracketed by CUDA events behind a GPU-side delay so that the host has finished enqueueing before the
device reaches the timed call; ``speedup`` is the geometric mean of mapping0/mapping1 per pair. Because
both arms are the same kernel here, ``speedup`` isolates the handoff; the absolute figures the
reference never published are added: TFLOP/s for prefill (``4*B*32*T^2*128/2`` FLOPs) and HBM GB/s for
decode (every attended K/V row once, Q, O, LSE and the appended rows).
"""
from __future__ import annotations

import argparse
import json
from dataclasses import dataclass, field
from pathlib import Path
from statistics import geometric_mean, median
from time import perf_counter_ns
from typing import Callable

from .cuda_runtime import build_cuda, cuda_device

HEADS_Q, HEADS_KV, HEAD_DIM = 32, 8, 128
SEED = 7911
RESOURCE_FIELDS = ("threads", "dynamic_shared_bytes", "static_shared_bytes", "registers_per_thread",
                   "local_bytes_per_thread", "binary_version", "ptx_version", "active_ctas_per_sm")


@dataclass
class Arm:
    """One mapping of one shape: the call that is timed, an untimed call that restores whatever state
    the timed call needs (decode: the step before it), and the outputs the timed call produces."""

    call: Callable[[], None]
    prepare: Callable[[], None]
    outputs: tuple


@dataclass
class Shape:
    """Everything the driver needs for one (batch, length) point."""

    arms: list
    resources: dict
    work: dict = field(default_factory=dict)  # {"flops": ...} or {"bytes": ...}


def _bits_equal(torch, left, right) -> bool:
    views = (torch.int16, torch.int32)  # O is BF16, LSE is FP32
    return all(torch.isfinite(b).all() and torch.equal(a.view(kind), b.view(kind))
               for a, b, kind in zip(left, right, views, strict=True))


def _require_same_bits(torch, left, right):
    if not _bits_equal(torch, left, right):
        raise RuntimeError("O or LSE differs between the dedicated-staging and the handoff schedule")


def _named_resources(values) -> dict:
    return {name: values[12 + index] for index, name in enumerate(RESOURCE_FIELDS)}


def _buffers(torch, sizes, device):
    return [torch.empty(count, device=device, dtype=torch.float32) for count in sizes[1:3]]


def prefill_shape(torch, ops, draw, batch: int, tokens: int) -> Shape:
    q = draw(batch, tokens, HEADS_Q, HEAD_DIM)
    k = draw(batch, tokens, HEADS_KV, HEAD_DIM)
    v = draw(batch, tokens, HEADS_KV, HEAD_DIM)
    scale = HEAD_DIM ** -0.5
    shape = Shape(arms=[], resources=_named_resources(ops.resources(q, k, v, 0, 1, True)),
                  work={"flops": 4.0 * batch * HEADS_Q * tokens * tokens * HEAD_DIM / 2})
    for mapping in (0, 1):
        out = torch.empty_like(q)
        lse = torch.empty((batch, HEADS_Q, tokens), device=q.device, dtype=torch.float32)
        scratch = _buffers(torch, ops.workspace_spec(q, k, v, 0, mapping, True), q.device)

        def call(out=out, lse=lse, scratch=scratch, mapping=mapping):
            ops.forward_out(q, k, v, out, lse, *scratch, 0, mapping, scale, True)

        call()
        shape.arms.append(Arm(call=call, prepare=lambda: None, outputs=(out, lse)))
    _require_same_bits(torch, shape.arms[0].outputs, shape.arms[1].outputs)
    return shape


def decode_shape(torch, ops, draw, batch: int, history: int) -> Shape:
    """Two consecutive decode steps on a cache with ``history`` valid rows and room for two more; the
    second step is the timed call, the first one re-primes the cache row it depends on."""
    old_k, old_v = draw(batch, history, HEADS_KV, HEAD_DIM), draw(batch, history, HEADS_KV, HEAD_DIM)
    tokens = [(draw(batch, 1, HEADS_Q, HEAD_DIM), draw(batch, 1, HEADS_KV, HEAD_DIM), draw(batch, 1, HEADS_KV, HEAD_DIM))
              for _ in range(2)]
    device = old_k.device
    lengths = [torch.full((batch,), history + step, dtype=torch.int32, device=device) for step in range(2)]
    shape = Shape(arms=[], resources={})
    first_step_outputs = []
    for mapping in (0, 1):
        kcache = torch.empty((batch, history + 2, HEADS_KV, HEAD_DIM), dtype=old_k.dtype, device=device)
        vcache = torch.empty_like(kcache)
        kcache[:, :history] = old_k
        vcache[:, :history] = old_v
        steps = []
        for step, (q, knew, vnew) in enumerate(tokens):
            out = torch.empty_like(q)
            lse = torch.empty((batch, HEADS_Q, 1), dtype=torch.float32, device=device)
            scratch = _buffers(torch, ops.workspace_spec(q, kcache, lengths[step], 0, mapping, True), device)

            def call(q=q, knew=knew, vnew=vnew, old=lengths[step], out=out, lse=lse, scratch=scratch,
                     kcache=kcache, vcache=vcache, mapping=mapping):
                ops.forward_out(q, kcache, vcache, knew, vnew, old, out, lse, *scratch, 0, mapping, True)

            call()
            steps.append((call, (out, lse)))
        expectations = [(old_k, kcache[:, :history]), (old_v, vcache[:, :history])]
        for step, (_, knew, vnew) in enumerate(tokens):
            row = slice(history + step, history + step + 1)
            expectations += [(knew, kcache[:, row]), (vnew, vcache[:, row])]
        if not all(torch.equal(want.view(torch.int16), got.view(torch.int16)) for want, got in expectations):
            raise RuntimeError("Fused append changed historical or newly appended KV")
        first_step_outputs.append(steps[0][1])
        shape.arms.append(Arm(call=steps[1][0], prepare=steps[0][0], outputs=steps[1][1]))
        if mapping == 1:
            shape.resources = _named_resources(ops.resources(tokens[1][0], kcache, lengths[1], 0, 1, True))
    _require_same_bits(torch, *first_step_outputs)
    _require_same_bits(torch, shape.arms[0].outputs, shape.arms[1].outputs)
    attended = history + 2  # rows visible to the timed (second) step
    row_bytes = HEADS_KV * HEAD_DIM * 2
    shape.work = {"bytes": 2 * batch * attended * row_bytes + 2 * batch * HEADS_Q * HEAD_DIM * 2
                  + batch * HEADS_Q * 4 + 4 * batch * row_bytes}
    return shape


class GuardedTimer:
    """Device time of one call, measured so that host enqueue latency cannot leak into it.

    A ~1 ms device-side delay is queued first; the start event, the call and the end event are enqueued
    behind it. If the delay had already drained when the host finished enqueueing (the gap between the
    lead event and the start event is shorter than the host needed), the sample is refused rather than
    reported: the reference's guard (``bench_operator.py:81-95``).
    """

    DELAY_CYCLES = 2_000_000

    def __init__(self, torch):
        self.torch = torch

    def microseconds(self, arm: Arm) -> float:
        torch = self.torch
        lead = torch.cuda.Event(enable_timing=True)
        begin = torch.cuda.Event(enable_timing=True)
        finish = torch.cuda.Event(enable_timing=True)
        arm.prepare()
        lead.record()
        host_start = perf_counter_ns()
        torch.cuda._sleep(self.DELAY_CYCLES)
        begin.record()
        arm.call()
        finish.record()
        host_ns = perf_counter_ns() - host_start
        finish.synchronize()
        if lead.elapsed_time(begin) * 1e6 <= host_ns:
            raise RuntimeError("The GPU reached the timed region before the host finished enqueueing")
        return begin.elapsed_time(finish) * 1e3


def time_shape(torch, shape: Shape, rounds: int, device) -> dict:
    """Alternating paired samples of the two arms; returns the timing part of a row."""
    for _ in range(4):  # warm both arms
        for arm in shape.arms:
            arm.prepare()
            arm.call()
    torch.cuda.synchronize(device)
    timer = GuardedTimer(torch)
    windows = []
    for index in range(rounds):
        order = (0, 1) if index % 2 == 0 else (1, 0)
        sample = {}
        for which in order:
            sample["default_us" if which == 0 else "candidate_us"] = timer.microseconds(shape.arms[which])
        windows.append({"default_us": sample["default_us"], "candidate_us": sample["candidate_us"]})
    typical = median(window["candidate_us"] for window in windows)
    timing = {"windows": windows, "candidate_us": typical,
              "speedup": geometric_mean(window["default_us"] / window["candidate_us"] for window in windows)}
    if "flops" in shape.work:
        timing["tflops"] = shape.work["flops"] / typical / 1e6
    if "bytes" in shape.work:
        timing["hbm_gbs"] = shape.work["bytes"] / typical / 1e3
    return timing


def parse_arguments(argv=None):
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--phase", required=True, choices=("prefill", "decode"))
    parser.add_argument("--source", type=Path, help="directory emitted earlier by tilecadence_b200.operator")
    parser.add_argument("--flash-attention-root", type=Path,
                        help="ignored: the sm_100a kernels need no FlashAttention checkout")
    parser.add_argument("--work", required=True, type=Path)
    parser.add_argument("--device", default="cuda:0")
    parser.add_argument("--batches", nargs="+", type=int, choices=(1, 4), default=(1, 4))
    parser.add_argument("--lengths", nargs="+", type=int, default=(128, 2048, 8192))
    parser.add_argument("--rounds", type=int, default=7)
    parser.add_argument("--verify-only", action="store_true")
    arguments = parser.parse_args(argv)
    if arguments.rounds < 2 or any(not 128 <= length <= 32768 for length in arguments.lengths):
        parser.error("Lengths must be in [128, 32768] and rounds must be at least two")
    return arguments


def main(argv=None):
    arguments = parse_arguments(argv)
    import torch

    arguments.work.mkdir(parents=True, exist_ok=False)
    source = arguments.source
    if source is None:
        from .operator import emit

        source = arguments.work / "source"
        emit(arguments.phase, source)
    device, _ = cuda_device(arguments.device)
    make_shape = {"prefill": prefill_shape, "decode": decode_shape}[arguments.phase]
    with torch.cuda.device(device), torch.inference_mode():
        ops, identity = build_cuda(source, arguments.flash_attention_root, device)
        generator = torch.Generator(device=device).manual_seed(SEED)

        def draw(*dims):
            return torch.randn(dims, generator=generator, device=device, dtype=torch.bfloat16)

        with (arguments.work / "rows.jsonl").open("x", encoding="utf-8") as log:
            for batch in arguments.batches:
                for length in arguments.lengths:
                    shape = make_shape(torch, ops, draw, batch, length)
                    row = {"phase": arguments.phase, "batch": batch, "length": length, "bitwise": True,
                           "resources": shape.resources}
                    if not arguments.verify_only:
                        row.update(time_shape(torch, shape, arguments.rounds, device))
                    if ops.library.device_status(device.index) != 0:
                        raise RuntimeError("A kernel reported an expired wait")
                    text = json.dumps(row)
                    log.write(text + "\n")
                    log.flush()
                    print(text, flush=True)
    (arguments.work / "build.json").write_text(json.dumps(identity, indent=2) + "\n", encoding="utf-8")


if __name__ == "__main__":
    main()

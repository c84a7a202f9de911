"""Check and time the generated two-tile attention residency schedules on a B200.

Same procedure as ``tilecadence/bench_exchange.py`` (``_reference`` :54-60, ``_assert_close`` :63-66,
``_validate`` :96-113, graph timing :116-163, ``run`` :194-232): every arm is solved, emitted and built;
the ``retain`` arm is compared with fp32 torch attention on the same device tensors (atol/rtol 0.003/0.01
FP16, 0.02/0.02 BF16; LSE 5e-4/1e-4) and every exchange arm must equal ``retain`` bit for bit; then each
arm is timed by replaying a CUDA graph of ``GRAPH_CALLS`` launches, once on one repeated buffer set and
once rotating over ``--slots`` sets. There is no stock-FlashAttention arm: the build has a single backend.
"""
import argparse
import json
from pathlib import Path
from statistics import median

from . import exchange, model
from .cuda_runtime import build_cuda, cuda_device
from .emit_exchange import RESOURCE_KEYS, emit

EXCHANGE_ARMS = ("one", "multi", "relocated_two_p")
GRAPH_CALLS = 16
REPLAYS = 32


def _reference(torch, slot, causal):
    q, k, v = (tensor.transpose(1, 2).float() for tensor in slot[:3])
    scores = (q @ k.transpose(-2, -1)) * (128 ** -0.5)
    if causal:
        index = torch.arange(q.size(2), device=q.device)
        scores.masked_fill_(index[None, :] > index[:, None], float("-inf"))
    return (scores.softmax(dim=-1) @ v).transpose(1, 2), scores.logsumexp(dim=-1)


def _assert_close(torch, actual, expected, dtype):
    atol, rtol = (0.003, 0.01) if dtype == torch.float16 else (0.02, 0.02)
    torch.testing.assert_close(actual[0].float(), expected[0].float(), atol=atol, rtol=rtol)
    torch.testing.assert_close(actual[1], expected[1], atol=0.0005, rtol=0.0001)


def _make_slots(torch, args, dtype, device):
    generator = torch.Generator(device=device).manual_seed(args.seed)
    shape = (args.batch, 64, args.heads, 128)
    slots = []
    for _ in range(args.slots):
        qkv = tuple(torch.randn(shape, dtype=dtype, device=device, generator=generator) for _ in range(3))
        slots.append((*qkv, torch.empty_like(qkv[0]),
                      torch.empty((args.batch, args.heads, 64), device=device, dtype=torch.float32)))
    return slots


def _forward(ops, causal):
    def forward(slot):
        q, k, v, out, lse = slot
        ops.forward_out(q, k, v, out, lse, None, causal, True, False)
        return out, lse

    return forward


def _validate(torch, arms, slots, causal, dtype):
    for slot in slots:
        reference = _reference(torch, slot, causal)
        retain = tuple(tensor.clone() for tensor in arms["retain"](slot))
        _assert_close(torch, retain, reference, dtype)
        for name, forward in arms.items():
            if name == "retain":
                continue
            actual = forward(slot)
            if not all(torch.equal(a.view(integer), b.view(integer))
                       for a, b, integer in zip(actual, retain, (torch.int16, torch.int32), strict=True)):
                raise RuntimeError(f"{name} differs bitwise from the retain schedule")


def _time_graph(torch, forward, slots, rotating):
    order = [slots[i % len(slots)] if rotating else slots[0] for i in range(GRAPH_CALLS)]
    forward(slots[0])
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for slot in order:
                forward(slot)
    samples = []
    for _ in range(REPLAYS):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        end.record()
        end.synchronize()
        samples.append(start.elapsed_time(end) * 1000 / GRAPH_CALLS)
    return median(samples)


def run(args):
    import torch

    args.work.mkdir(parents=True, exist_ok=False)
    device, _ = cuda_device(args.device)
    dtype = torch.float16 if args.dtype == "float16" else torch.bfloat16
    rows = {}
    with torch.cuda.device(device), torch.inference_mode():
        arms, builds = {}, {}
        for arm in ("retain", *EXCHANGE_ARMS):
            problem = exchange.build_problem(arm)
            result = model.solve(problem, max_time_seconds=args.seconds)
            exchange.verify(problem.provenance[exchange.PROVENANCE_KEY], result)
            emit(problem, result, args.work / arm / "emitted")
            ops, builds[arm] = build_cuda(args.work / arm / "emitted", None, device)
            arms[arm] = _forward(ops, args.causal)
            rows[arm] = {"status": result["status"], "source_steps": result["finish_step"], "objective": result["objective"]}
        slots = _make_slots(torch, args, dtype, device)
        resources = dict(zip(RESOURCE_KEYS, ops.resources(slots[0][0], args.causal), strict=True))
        if resources["theoretical_active_ctas_per_sm"] < 1 or resources["diagnostic_guard"]:
            raise RuntimeError(f"Generated kernel cannot be used for benchmarking: {resources}")
        _validate(torch, arms, slots, args.causal, dtype)
        if ops.library.device_status(device.index) != 0:
            raise RuntimeError("A kernel reported an expired wait")
        if not args.verify_only:
            for arm, forward in arms.items():
                rows[arm]["repeated_us"] = _time_graph(torch, forward, slots, rotating=False)
                rows[arm]["rotating_us"] = _time_graph(torch, forward, slots, rotating=True)
            for arm in EXCHANGE_ARMS:
                for key in ("repeated_us", "rotating_us"):
                    rows[arm][key.replace("_us", "_speedup_vs_retain")] = rows["retain"][key] / rows[arm][key]
    record = {"dtype": args.dtype, "causal": args.causal, "batch": args.batch, "heads": args.heads, "slots": args.slots,
              "verified": True, "resources": resources, "arms": rows}
    (args.work / "result.json").write_text(json.dumps(record, indent=2) + "\n")
    (args.work / "build.json").write_text(json.dumps(builds, indent=2) + "\n")
    print(json.dumps(record), flush=True)
    return record


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--work", type=Path, required=True)
    parser.add_argument("--flash-attention-root", type=Path, help="Ignored: no FlashAttention checkout is needed")
    parser.add_argument("--device", default="cuda:0")
    parser.add_argument("--dtype", choices=("float16", "bfloat16"), default="float16")
    parser.add_argument("--causal", action="store_true")
    parser.add_argument("--batch", type=int, default=1)
    parser.add_argument("--heads", type=int, default=192)
    parser.add_argument("--slots", type=int, default=16)
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--seconds", type=float, default=2)
    parser.add_argument("--verify-only", action="store_true")
    args = parser.parse_args()
    if args.batch < 1 or args.heads < 1 or args.slots < 1:
        parser.error("batch, heads and slots must be positive")
    run(args)


if __name__ == "__main__":
    main()

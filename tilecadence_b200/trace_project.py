"""Time line of one launch of the QKV projection kernel inside a chain of launches, measured inside the kernel.

    python -m tilecadence_b200.trace_project [--build-only] [--device cuda:0] [--tokens 1]

Builds the projection kernel with the ``TC_TRACE`` switch (thread 0 and the producer lane of every CTA record
``%globaltimer`` at fixed points; see the list in ``csrc/project/qkv_rope_sm100.cu``), replays a captured chain of
16 launches over eight rotating weight sets (252 MB, more than L2 holds) and prints, for the last launch, every
recorded point as minimum / median / maximum over the CTAs in microseconds after the stream dependency resolved,
and the period of the chain. The trace build is a library of its own in the build cache; the shipped library never
contains the switch.
"""
from __future__ import annotations

import argparse
import ctypes
from pathlib import Path
import tempfile

POINTS = ("entry", "ring and L2 prefetch issued", "dependency resolved", "token slab ready", "tile 0 arrived",
          "first refilled tile arrived", "weight loop done", "cluster barrier passed", "head stored (rank 0)")


def build(verbose=False):
    """The projection phase library with the trace switch; compiled where nvcc is, found again by hash elsewhere."""
    from . import cuda_runtime

    with tempfile.TemporaryDirectory(prefix="tilecadence_b200_trace_") as scratch:
        target = Path(scratch) / "project"
        target.mkdir()
        for name, path in cuda_runtime.staged_sources("project").items():
            (target / name).write_bytes(Path(path).read_bytes())
        path, _ = cuda_runtime.compile_directory(target, verbose=verbose, defines=("TC_TRACE",))
    return path


def run(device="cuda:0", tokens=1, hidden=2560, sets=8, chain=16):
    import numpy as np
    import torch

    from . import cuda_runtime

    device, _ = cuda_runtime.cuda_device(device)
    library = cuda_runtime.load_library(build())
    ops = cuda_runtime.ops_for(library, "project")
    generator = torch.Generator(device=device).manual_seed(5)
    weights = [(torch.randn((48 * 128, hidden), generator=generator, device=device) / hidden ** 0.5).to(torch.bfloat16)
               for _ in range(sets)]
    x = torch.randn((tokens, hidden), generator=generator, device=device).to(torch.bfloat16)
    ones = torch.ones(128, device=device, dtype=torch.bfloat16)
    cos, sin = torch.rand((4096, 64), device=device), torch.rand((4096, 64), device=device)
    positions = torch.arange(tokens, device=device, dtype=torch.int32)
    outputs = [torch.empty((tokens, 1, heads, 128), device=device, dtype=torch.bfloat16) for heads in (32, 8, 8)]
    turn = [0]

    def step():
        ops.forward_out(x, weights[turn[0] % sets], positions, *outputs, q_norm_weight=ones, k_norm_weight=ones,
                        rope_cos=cos, rope_sin=sin)
        turn[0] += 1

    step()
    torch.cuda.synchronize(device)
    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        step()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(chain):
                step()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize(device)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    graph.replay()
    end.record()
    torch.cuda.synchronize(device)
    table = np.zeros((256, 16), dtype=np.uint64)
    library.handle.tc_debug_project_trace.argtypes = [ctypes.c_void_p]
    if library.handle.tc_debug_project_trace(table.ctypes.data) != 0:
        raise RuntimeError("tc_debug_project_trace failed")
    stamps = table[table[:, 0] != 0].astype(np.int64)
    origin = stamps[:, 2].min()
    print(f"{tokens} token(s), hidden {hidden}, {stamps.shape[0]} CTAs; period of the chain "
          f"{start.elapsed_time(end) / chain * 1e3:.2f} us; microseconds after the dependency resolved (min / median / max)")
    for slot, name in enumerate(POINTS):
        column = stamps[:, slot]
        column = column[column > 0]
        if column.size:
            print(f"  {name:30s} {(column.min() - origin) / 1e3:7.2f} {(np.median(column) - origin) / 1e3:7.2f} "
                  f"{(column.max() - origin) / 1e3:7.2f}")
    if library.device_status(device.index) != 0:
        raise RuntimeError("a kernel reported an expired wait")


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--build-only", action="store_true", help="compile the trace library and stop (needs no GPU)")
    parser.add_argument("--device", default="cuda:0")
    parser.add_argument("--tokens", type=int, default=1)
    arguments = parser.parse_args(argv)
    if arguments.build_only:
        print(build())
        return
    run(arguments.device, arguments.tokens)


if __name__ == "__main__":
    main()

"""Time line of a decode step, measured inside the kernel.

    python -m tilecadence_b200.trace_decode [--build-only] [--device cuda:0]

Builds the decode kernel with the ``TC_TRACE`` switch (thread 0 and the producer lane of every CTA record
``%globaltimer`` at fixed points; see the list in ``csrc/decode/decode_sm100.cu``), replays a captured chain
of config-4 steps (batch 1, 8192 of 32768 rows valid, eight rotating cache sets) without and with the
cache-stable promise, and prints for a few launches of the steady state, per recorded point, the
minimum / median / maximum over the launch's CTAs in microseconds since the launch's first CTA started.
The trace build is a library of its own in the build cache; the shipped library never contains the switch.
"""
from __future__ import annotations

import argparse
import ctypes
from pathlib import Path
import tempfile

POINTS = (("entry", 0), ("ready", 3), ("ring issued", 24), ("prefetch issued", 25), ("dependency resolved", 27),
          ("tile 0 arrived", 4), ("tile 0 consumed", 5), ("last tile issued", 26), ("key loop done", 20),
          ("partial staged", 21), ("ticket", 22), ("split LSEs loaded", 28), ("splits merged", 29), ("stored", 19))


def build(verbose=False):
    """The decode phase library with the trace switch; compiled where nvcc is, found again by hash elsewhere."""
    from . import cuda_runtime
    from .operator import emit

    with tempfile.TemporaryDirectory(prefix="tilecadence_b200_trace_") as scratch:
        emit("decode", Path(scratch) / "decode")
        path, _ = cuda_runtime.compile_directory(Path(scratch) / "decode", verbose=verbose, defines=("TC_TRACE",))
    return path


def run(device="cuda:0", launches=4, graph_steps=16, sets=8, capacity=32768, valid=8192):
    import numpy as np
    import torch

    from . import cuda_runtime

    device, _ = cuda_runtime.cuda_device(device)
    library = cuda_runtime.load_library(build())
    ops = cuda_runtime.ops_for(library, "decode")
    generator = torch.Generator(device=device).manual_seed(3)
    caches = [tuple(torch.randn((1, capacity, 8, 128), generator=generator, device=device, dtype=torch.bfloat16)
                    for _ in range(2)) for _ in range(sets)]
    q = torch.randn((1, 1, 32, 128), generator=generator, device=device, dtype=torch.bfloat16)
    knew, vnew = (torch.randn((1, 1, 8, 128), generator=generator, device=device, dtype=torch.bfloat16) for _ in range(2))
    old = torch.full((1,), valid, dtype=torch.int32, device=device)
    out, lse = torch.empty_like(q), torch.empty((1, 32, 1), device=device)
    spec = ops.workspace_spec(q, caches[0][0], old, 0, 1, True)
    workspace = [torch.empty(n, device=device) for n in spec[1:]]
    ctas = spec[0] * 8
    library.handle.tc_debug_trace.argtypes = [ctypes.c_void_p]
    for promise in (False, True):
        steps = [ops.bind_forward_out(q, kc, vc, knew, vnew, old, out, lse, *workspace, 0, 1, True, cache_stable=promise)
                 for kc, vc in caches]
        steps[0]()
        torch.cuda.synchronize(device)
        stream = torch.cuda.Stream(device)
        with torch.cuda.stream(stream):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for index in range(graph_steps):
                    steps[index % sets]()
        for _ in range(5):
            graph.replay()
        torch.cuda.synchronize(device)
        table = np.zeros((1024, 32), dtype=np.uint64)
        if library.handle.tc_debug_trace(table.ctypes.data) != 0:
            raise RuntimeError("tc_debug_trace failed")
        table = table.astype(np.int64)
        by_launch = {}
        for row in table:
            by_launch.setdefault(int(row[1]) // ctas, []).append(row)
        complete = sorted(key for key, rows in by_launch.items() if len(rows) == ctas)[-(launches + 1):-1]
        print(f"cache_stable={promise}: {ctas} CTAs per launch, min / median / max over CTAs, microseconds")
        previous = None
        for key in complete:
            rows = np.stack(by_launch[key])
            start = rows[:, 0].min()
            cells = []
            for name, column in POINTS:
                stamps = rows[:, column]
                stamps = stamps[stamps >= start]  # points a launch never reached keep an older launch's stamp
                if len(stamps):
                    rel = (stamps - start) / 1e3
                    cells.append(f"{name} {rel.min():.2f}/{np.median(rel):.2f}/{rel.max():.2f}")
            end = rows[:, [19, 22]].max()
            note = "" if previous is None else f" | period {(start - previous[0]) / 1e3:.2f}, start - previous end {(start - previous[1]) / 1e3:.2f}"
            print(f"  launch {key}: " + "; ".join(cells) + f"; end {(end - start) / 1e3:.2f}" + note)
            previous = (start, end)


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--build-only", action="store_true", help="compile the trace library and stop (needs no GPU)")
    parser.add_argument("--device", default="cuda:0")
    arguments = parser.parse_args(argv)
    if arguments.build_only:
        print(build(verbose=False))
        return
    run(arguments.device)


if __name__ == "__main__":
    main()

"""Time line of one prefill launch, measured inside the kernel.

    python -m tilecadence_b200.trace_prefill [--build-only] [--tokens 8192] [--batch 1] [--heads 32] [--cta 0]

Builds the prefill kernel with the ``TC_TRACE`` switch (one thread of each role logs (tag, ``%globaltimer``)
records; roles and tags are listed in ``csrc/prefill/prefill_sm100.cu``), runs one launch and prints, for one
CTA, every record of every role in microseconds since that CTA's first record, unit by unit; ``--cta -1`` prints
one line per CTA instead (its units, first and last record relative to the launch's first). The trace build is a
library of its own in the build cache; the shipped library never contains the switch.
"""
from __future__ import annotations

import argparse
import ctypes
from pathlib import Path
import tempfile

ROLES = ("producer", "score MMA", "PV head 0", "PV head 1", "softmax 0", "softmax 1")
TAGS = {1: "Q tile issued", 2: "first K/V issued", 3: "last K/V issued", 10: "first score MMA", 11: "last score MMA",
        20: "first PV", 21: "last PV", 30: "first scores arrived", 31: "key loop done", 32: "LSE left", 33: "last PV done",
        34: "rows stored"}


def build(verbose=False):
    from . import cuda_runtime
    from .operator import emit

    with tempfile.TemporaryDirectory(prefix="tilecadence_b200_trace_") as scratch:
        emit("prefill", Path(scratch) / "prefill")
        path, _ = cuda_runtime.compile_directory(Path(scratch) / "prefill", verbose=verbose, defines=("TC_TRACE",))
    return path


def run(device="cuda:0", batch=1, tokens=8192, cta=0, q_heads=32):
    import numpy as np
    import torch

    from . import cuda_runtime

    device, _ = cuda_runtime.cuda_device(device)
    library = cuda_runtime.load_library(build())
    ops = cuda_runtime.ops_for(library, "prefill", q_heads=q_heads)
    generator = torch.Generator(device=device).manual_seed(1)
    q = torch.randn((batch, tokens, q_heads, 128), generator=generator, device=device, dtype=torch.bfloat16)
    k, v = (torch.randn((batch, tokens, q_heads // 4, 128), generator=generator, device=device, dtype=torch.bfloat16)
            for _ in range(2))
    out, lse = torch.empty_like(q), torch.empty((batch, q_heads, tokens), device=device)
    empty = torch.empty(0, device=device)
    for _ in range(3):
        ops.forward_out(q, k, v, out, lse, empty, empty, 0, 1, 128 ** -0.5, True)
    torch.cuda.synchronize(device)
    if library.handle.tc_debug_prefill_trace_clear() != 0:
        raise RuntimeError("tc_debug_prefill_trace_clear failed")
    ops.forward_out(q, k, v, out, lse, empty, empty, 0, 1, 128 ** -0.5, True)
    torch.cuda.synchronize(device)
    table = np.zeros((148, len(ROLES), 256), dtype=np.uint64)
    library.handle.tc_debug_prefill_trace.argtypes = [ctypes.c_void_p]
    if library.handle.tc_debug_prefill_trace(table.ctypes.data) != 0:
        raise RuntimeError("tc_debug_prefill_trace failed")
    everything = table[table != 0] >> np.uint64(8)
    first, last = int(everything.min()), int(everything.max())
    if cta < 0:
        print(f"batch {batch}, {tokens} tokens, {q_heads} query heads; whole launch {(last - first) / 1e3:.1f} us; per CTA: "
              "units, first record, last record (us since the launch's first record)")
        for index in range(table.shape[0]):
            stamps = table[index][table[index] != 0] >> np.uint64(8)
            if stamps.size:
                units = int(((table[index, 0] & np.uint64(0xFF)) == 1).sum())
                print(f"  CTA {index:3d}: {units:3d} units {(int(stamps.min()) - first) / 1e3:8.2f} {(int(stamps.max()) - first) / 1e3:8.2f}")
        return
    records = []
    for role, name in enumerate(ROLES):
        for word in table[cta, role]:
            word = int(word)
            if word:
                records.append((word >> 8, name, TAGS.get(word & 0xFF, str(word & 0xFF))))
    records.sort()
    start = records[0][0]
    print(f"batch {batch}, {tokens} tokens, {q_heads} query heads; whole launch {(last - first) / 1e3:.1f} us; "
          f"CTA {cta}, microseconds since its first record")
    for stamp, name, tag in records:
        print(f"  {(stamp - start) / 1e3:9.2f}  {name:10s} {tag}")


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--build-only", action="store_true", help="compile the trace library and stop (needs no GPU)")
    parser.add_argument("--device", default="cuda:0")
    parser.add_argument("--batch", type=int, default=1)
    parser.add_argument("--tokens", type=int, default=8192)
    parser.add_argument("--heads", type=int, default=32)
    parser.add_argument("--cta", type=int, default=0)
    arguments = parser.parse_args(argv)
    if arguments.build_only:
        print(build())
        return
    run(arguments.device, arguments.batch, arguments.tokens, arguments.cta, arguments.heads)


if __name__ == "__main__":
    main()

"""Generate the golden attention vectors from the reference's own CPU attention.

Run where the reference tree is available:

    python tests/golden/make_golden.py /path/to/TileCadence

It imports ``tilecadence.bench_exchange._reference`` (``bench_exchange.py:54-60``) from that tree,
feeds it small seeded inputs and stores, in ``attention_golden.npz``, a SHA-256 of the input words
(the inputs themselves are regenerated from the seed by ``golden_inputs``), the full fp32 LSE, the
fp32 O rows of every ``stride``-th token, and float64 sum / absolute-sum checksums of the whole O. ``_reference`` has equal head counts and no KV cache, so the GQA cases
repeat each KV head four times before the call and the decode cases pass the visible prefix of
the cache (new row included) with a single query row and no causal mask; that is exactly the
arithmetic the reference's CUDA path is checked against in its own benchmarks.
"""
import importlib.util
from pathlib import Path
import sys
import types

import numpy as np
import torch


def load_reference(root):
    root = Path(root)
    package = types.ModuleType("tilecadence_reference")
    package.__path__ = [str(root / "tilecadence")]
    sys.modules["tilecadence_reference"] = package
    for name in ("cuda_runtime", "bench_exchange"):
        spec = importlib.util.spec_from_file_location(f"tilecadence_reference.{name}", root / "tilecadence" / f"{name}.py")
        module = importlib.util.module_from_spec(spec)
        sys.modules[spec.name] = module
        spec.loader.exec_module(module)
    return sys.modules["tilecadence_reference.bench_exchange"]._reference


def words(tensor):
    return tensor.contiguous().view(torch.int16).numpy()


def digest(*tensors):
    from hashlib import sha256

    state = sha256()
    for tensor in tensors:
        state.update(words(tensor).tobytes())
    return np.frombuffer(state.digest(), dtype=np.uint8)


def golden_inputs(case):
    """Seeded inputs of one golden case; shared with the tests so both sides draw the same bits."""
    if case == "two_tile":
        generator = torch.Generator().manual_seed(0)
        return tuple(normal(generator, (1, 64, 8, 128), torch.float16) for _ in range(3))
    if case == "prefill":
        generator = torch.Generator().manual_seed(1)
        q = normal(generator, (1, 192, 8, 128), torch.bfloat16)
        k, v = (normal(generator, (1, 192, 2, 128), torch.bfloat16) for _ in range(2))
        return q, k, v
    if case == "decode":
        generator = torch.Generator().manual_seed(3)
        kcache, vcache = (normal(generator, (2, 200, 2, 128), torch.bfloat16) for _ in range(2))
        q = normal(generator, (2, 1, 8, 128), torch.bfloat16)
        knew, vnew = (normal(generator, (2, 1, 2, 128), torch.bfloat16) for _ in range(2))
        return kcache, vcache, q, knew, vnew, torch.tensor([130, 7], dtype=torch.int32)
    raise KeyError(case)


STRIDES = {"two_tile": 4, "prefill": 6, "decode": 1}


def record(arrays, case, inputs, out, lse):
    out = out.contiguous()
    arrays[f"{case}_inputs_sha256"] = digest(*inputs)
    arrays[f"{case}_o_rows"] = out[:, ::STRIDES[case]].contiguous().numpy()
    arrays[f"{case}_o_checksum"] = np.array([out.double().sum().item(), out.double().abs().sum().item()])
    arrays[f"{case}_lse"] = lse.contiguous().numpy()


def normal(generator, shape, dtype):
    return torch.randn(shape, generator=generator, dtype=torch.float32).to(dtype)


def main():
    if len(sys.argv) != 2:
        sys.exit(f"usage: python {sys.argv[0]} /path/to/TileCadence")
    reference = load_reference(sys.argv[1])
    arrays = {}

    # Two-tile exchange config: batch 1, 8 heads, 64 tokens, fp16, non-causal, seed 0.
    q, k, v = golden_inputs("two_tile")
    record(arrays, "two_tile", (q, k, v), *reference(torch, (q, k, v), False))

    # Causal GQA prefill, bf16, 8 query heads over 2 KV heads, 192 tokens (one full and one ragged tile).
    q, k, v = golden_inputs("prefill")
    record(arrays, "prefill", (q, k, v),
           *reference(torch, (q, k.repeat_interleave(4, dim=2), v.repeat_interleave(4, dim=2)), True))

    # Decode with append: batch 2, capacity 200, old lengths 130 and 7, 8 query heads over 2 KV heads.
    kcache, vcache, q, knew, vnew, old = golden_inputs("decode")
    outs, lses = [], []
    for b, length in enumerate(old.tolist()):
        kvis = torch.cat([kcache[b:b + 1, :length], knew[b:b + 1]], dim=1).repeat_interleave(4, dim=2)
        vvis = torch.cat([vcache[b:b + 1, :length], vnew[b:b + 1]], dim=1).repeat_interleave(4, dim=2)
        out, lse = reference(torch, (q[b:b + 1], kvis, vvis), False)
        outs.append(out)
        lses.append(lse)
    record(arrays, "decode", (kcache, vcache, q, knew, vnew), torch.cat(outs), torch.cat(lses))

    target = Path(__file__).with_name("attention_golden.npz")
    np.savez_compressed(target, **arrays)
    print(target, target.stat().st_size, "bytes")


if __name__ == "__main__":
    main()

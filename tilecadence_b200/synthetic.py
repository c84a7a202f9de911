"""Seeded synthetic inputs for the benchmarks.

The reference's harness draws its tensors from one seeded generator in a fixed order
(``tilecadence/bench_operator.py:124-127``: q, then k, then v; decode prefix K, prefix V, then per step
q, k, v). The draws here are made on the CPU, so that a host-side checker sees the same bits as the
device, and stand in for the saved model projections the reference measured on.
"""
from __future__ import annotations


def seeded_normal(seed, *shapes, dtype=None):
    """N(0,1) tensors drawn in order from one CPU generator seeded with ``seed`` and cast to ``dtype``
    (BF16 by default)."""
    import torch

    generator = torch.Generator().manual_seed(seed)
    dtype = torch.bfloat16 if dtype is None else dtype
    return [torch.randn(shape, generator=generator, dtype=torch.float32).to(dtype) for shape in shapes]

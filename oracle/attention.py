"""CPU oracle for the attention hot path. TEST INFRASTRUCTURE ONLY.

Nothing in the product path may import this module; only ``tests/``, ``__graft_entry__.smoke()``
and the CPU-baseline legs of ``bench.py`` use it, as the checker or as the timed CPU arm.

It restates, in fp32 torch on the host, the only CPU-capable attention the reference ships:
``tilecadence/bench_exchange.py:54-60`` (``_reference``): transpose to [B,H,S,D], fp32,
``scores = q @ k^T * scale``, causal ``masked_fill(col > row, -inf)``, ``softmax @ v`` and
``logsumexp``. On top of that come the conventions the reference's CUDA path adds:

* GQA: query head ``h`` reads KV head ``h // 4`` (``long_prefill_rowblock.cuh:219,225``; decode row
  mapping ``cuda/decode/decode.cu:97-105``);
* decode visibility: keys ``[0, old_len + 1)`` after the append, ``[0, old_len)`` without, no causal
  mask (``cuda/prefill/common.cuh:49``, ``ab_fused_splitkv.cuh:36,231``), scale 128^-0.5
  (``decode.cu:106``); the append is a bit copy of the new row into row ``old_len``
  (``ab_fused_splitkv.cuh:189-212``);
* LSE is the natural-log ``m*scale + ln(sum)`` (``cuda/exchange/backend.cuh:417``); a row with no
  visible key gives O = 0 and LSE = +inf in a final result, -inf in a split partial
  (``ab_fused_splitkv.cuh:82,322``);
* split merge: ``LSE = ln sum_s exp(LSE_s)``, ``O = sum_s exp(LSE_s - LSE) O_s`` (the combine kernel
  launched at ``decode.cu:131-140``).

Pinned against outputs of the reference's own ``_reference`` (imported from the reference tree when
the fixtures were generated): see ``tests/golden/make_golden.py`` and ``tests/test_oracle_golden.py``.
The reference stores no golden vectors of its own for this path.
"""
from __future__ import annotations

import math

import torch

GROUP = 4  # query heads per KV head
DIM = 128
DEFAULT_SCALE = DIM ** -0.5


def seeded_normal(seed, *shapes, dtype=torch.bfloat16):
    """N(0,1) tensors drawn in order from one CPU generator and cast to ``dtype``."""
    generator = torch.Generator().manual_seed(seed)
    return [torch.randn(shape, generator=generator, dtype=torch.float32).to(dtype) for shape in shapes]


def attention(q, k, v, causal, scale=DEFAULT_SCALE, row_block=1024):
    """O [B,Sq,Hq,D] fp32 and LSE [B,Hq,Sq] fp32 for BSHD inputs; KV heads are shared by groups.

    ``bench_exchange.py:54-60`` evaluated per KV head and per block of query rows so that the
    score matrix stays small at long sequence lengths. Causal alignment is top-left with
    ``Sq == Sk`` (the prefill contract).
    """
    batch, sq, hq, dim = q.shape
    sk, hkv = k.shape[1], k.shape[2]
    assert hq % hkv == 0 and v.shape == k.shape and (not causal or sq == sk)
    group = hq // hkv
    out = torch.empty((batch, sq, hq, dim), dtype=torch.float32)
    lse = torch.empty((batch, hq, sq), dtype=torch.float32)
    for b in range(batch):
        for g in range(hkv):
            kh = k[b, :, g].float()  # [Sk, D]
            vh = v[b, :, g].float()
            qh = q[b, :, g * group:(g + 1) * group].float().permute(1, 0, 2)  # [group, Sq, D]
            for r0 in range(0, sq, row_block):
                r1 = min(sq, r0 + row_block)
                visible = r1 if causal else sk
                scores = (qh[:, r0:r1] @ kh[:visible].T) * scale  # [group, rows, visible]
                if causal:
                    rows = torch.arange(r0, r1)[:, None]
                    cols = torch.arange(visible)[None, :]
                    scores.masked_fill_(cols > rows, float("-inf"))
                lse[b, g * group:(g + 1) * group, r0:r1] = scores.logsumexp(dim=-1)
                out[b, r0:r1, g * group:(g + 1) * group] = (scores.softmax(dim=-1) @ vh[:visible]).permute(1, 0, 2)
    return out, lse


def decode_step(q, kcache, vcache, knew, vnew, old_lengths, append=True, scale=DEFAULT_SCALE,
                shard_start=0, partial=False):
    """One decode step on host tensors; returns (O, LSE, kcache_after, vcache_after).

    q [B,1,Hq,D]; caches [B,C,Hkv,D] holding global rows [shard_start, shard_start + C);
    knew/vnew [B,1,Hkv,D]; old_lengths int [B] (global). O is fp32 [B,1,Hq,D], LSE fp32 [B,Hq,1].
    With ``partial`` an empty row gets LSE = -inf (a split partial) instead of +inf.
    """
    batch, _, hq, dim = q.shape
    capacity, hkv = kcache.shape[1], kcache.shape[2]
    group = hq // hkv
    kcache, vcache = kcache.clone(), vcache.clone()
    out = torch.zeros((batch, 1, hq, dim), dtype=torch.float32)
    lse = torch.empty((batch, hq, 1), dtype=torch.float32)
    for b in range(batch):
        old = int(old_lengths[b])
        row = old - shard_start
        if append and 0 <= row < capacity:
            kcache[b, row] = knew[b, 0]
            vcache[b, row] = vnew[b, 0]
        visible = min(max(old + (1 if append else 0) - shard_start, 0), capacity)
        if visible == 0:
            lse[b] = float("-inf") if partial else float("inf")
            continue
        for g in range(hkv):
            qh = q[b, 0, g * group:(g + 1) * group].float()  # [group, D]
            scores = (qh @ kcache[b, :visible, g].float().T) * scale
            lse[b, g * group:(g + 1) * group, 0] = scores.logsumexp(dim=-1)
            out[b, 0, g * group:(g + 1) * group] = scores.softmax(dim=-1) @ vcache[b, :visible, g].float()
    return out, lse, kcache, vcache


def rope_tables(positions, theta=1.0e6, dim=64):
    """cos / sin tables fp32 [positions, dim] of rotary position embedding with base ``theta`` (Qwen3's
    1e6 by default): angle[p, i] = p * theta ** (-i / dim), computed in float64 and rounded once."""
    inv_freq = theta ** (-torch.arange(dim, dtype=torch.float64) / dim)
    angle = torch.arange(positions, dtype=torch.float64)[:, None] * inv_freq[None]
    return angle.cos().float(), angle.sin().float()


def rope_rotate(x, cos, sin):
    """Rotate-half RoPE of x [..., 128] (any float dtype) with cos/sin [..., 64] broadcastable to it:
    x'[i] = x[i]*cos[i] - x[i+64]*sin[i], x'[i+64] = x[i+64]*cos[i] + x[i]*sin[i], each product and sum
    a separate fp32 rounding, result rounded to x's dtype. The published rotate-half form (the one
    Qwen-style models use); the reference itself receives q and K already rotated
    (``tilecadence/cuda/decode/ab_fused_splitkv.cuh:189``)."""
    lo, hi = x[..., :64].float(), x[..., 64:].float()
    out_lo = lo * cos - hi * sin
    out_hi = hi * cos + lo * sin
    return torch.cat([out_lo, out_hi], dim=-1).to(x.dtype)


def project_qkv_rope(x, w_qkv, positions, q_heads, kv_heads, q_norm_weight=None, k_norm_weight=None, cos=None,
                     sin=None, rms_eps=1e-6):
    """The step before decode attention for one new token per sequence: y = x W^T in fp32, per-head RMS
    norm of the q and k heads (x * rsqrt(mean(x^2) + eps) rounded to the input dtype, times the weight,
    rounded again: the form Qwen3 uses), rotate-half RoPE of q and k for ``positions``, v untouched.

    x [tokens, hidden], w_qkv [(q_heads + 2 kv_heads) * 128, hidden], rows ordered q, k, v heads.
    Returns q [tokens,1,q_heads,128], knew and vnew [tokens,1,kv_heads,128] in x's dtype. The reference
    has no such step (its decode op receives these tensors); this restates the published model math.
    """
    tokens = x.size(0)
    y = (x.float() @ w_qkv.float().T).view(tokens, q_heads + 2 * kv_heads, 128)

    def normed(part, weight):
        if weight is None:
            return part.to(x.dtype)
        scaled = part * torch.rsqrt(part.pow(2).mean(-1, keepdim=True) + rms_eps)
        return (scaled.to(x.dtype).float() * weight.float()).to(x.dtype)

    q = normed(y[:, :q_heads], q_norm_weight)
    k = normed(y[:, q_heads:q_heads + kv_heads], k_norm_weight)
    v = y[:, q_heads + kv_heads:].to(x.dtype)
    if cos is not None:
        position = positions.long().clamp(0, cos.size(0) - 1)
        c, s = cos[position][:, None, :], sin[position][:, None, :]
        q, k = rope_rotate(q, c, s), rope_rotate(k, c, s)
    return q[:, None], k[:, None], v[:, None]


def decode_step_rope(q, kcache, vcache, knew, vnew, old_lengths, cos, sin, append=True, scale=DEFAULT_SCALE):
    """:func:`decode_step` on un-rotated q / knew: both are rotated for position ``old_lengths[b]``
    (clamped to the table), rounded to their dtype, and the step runs on the rotated tensors."""
    position = old_lengths.long().clamp(0, cos.size(0) - 1)
    c, s = cos[position][:, None, None, :], sin[position][:, None, None, :]  # [B,1,1,64]
    return decode_step(rope_rotate(q, c, s), kcache, vcache, rope_rotate(knew, c, s), vnew, old_lengths, append, scale)


def decode_step_indexed(q, kcache, vcache, knew, vnew, old_lengths, block_table=None, cache_batch_idx=None,
                        append=True, scale=DEFAULT_SCALE):
    """Decode step over indexed caches, by gathering each sequence's rows into a contiguous cache,
    running :func:`decode_step` and scattering the caches back.

    Follows the two indirections of ``tilecadence/cuda/decode/ab_fused_splitkv.cuh:92-103``:
    with ``block_table`` int [B, pages] the caches are pages [P, page_size, Hkv, D] and row ``r`` of
    sequence ``b`` is row ``r % page_size`` of page ``block_table[b, r // page_size]``; with
    ``cache_batch_idx`` int [B] sequence ``b`` uses cache entry ``cache_batch_idx[b]``.
    Returns (O, LSE, kcache_after, vcache_after) in the caches' own layout.
    """
    if (block_table is None) == (cache_batch_idx is None):
        raise ValueError("pass exactly one of block_table / cache_batch_idx")
    if block_table is not None:
        index = block_table.long()
        gather = lambda cache: cache[index].flatten(1, 2)  # [B, pages * page_size, Hkv, D]
    else:
        index = cache_batch_idx.long()
        gather = lambda cache: cache[index]
    out, lse, k_seq, v_seq = decode_step(q, gather(kcache), gather(vcache), knew, vnew, old_lengths, append, scale)
    k_after, v_after = kcache.clone(), vcache.clone()
    if block_table is not None:
        page = kcache.shape[1]
        k_after[index] = k_seq.unflatten(1, (-1, page))
        v_after[index] = v_seq.unflatten(1, (-1, page))
    else:
        k_after[index] = k_seq
        v_after[index] = v_seq
    return out, lse, k_after, v_after


def combine(partial_o, partial_lse):
    """Merge ``parts`` partial results: partial_o [parts, rows, D] fp32, partial_lse [parts, rows].

    Returns O [rows, D] fp32 and LSE [rows] (+inf where no part contributed).
    """
    lse_max = partial_lse.max(dim=0).values
    safe_max = torch.where(torch.isinf(lse_max), torch.zeros_like(lse_max), lse_max)
    weights = torch.exp(partial_lse - safe_max[None])
    weights = torch.where(torch.isinf(partial_lse) & (partial_lse < 0), torch.zeros_like(weights), weights)
    total = weights.sum(dim=0)
    safe_o = torch.where(weights[..., None] > 0, partial_o, torch.zeros_like(partial_o))
    merged = (weights[..., None] * safe_o).sum(dim=0) / torch.where(total > 0, total, torch.ones_like(total))[..., None]
    lse = torch.where(total > 0, safe_max + torch.log(total), torch.full_like(total, float("inf")))
    return merged, lse


def check_outputs(actual_o, actual_lse, expected_o, expected_lse, dtype=torch.bfloat16):
    """The acceptance bar: max-abs O error <= 2e-2 (BF16) / 1e-2 (FP16), LSE <= 1e-3 relative.

    "Relative" needs a floor, because an LSE can be exactly 0: the error is divided by max(|LSE|, 0.1), so
    the bound is the relative one wherever |LSE| >= 0.1 and 1e-4 absolute below that.
    Returns the two measured errors; raises AssertionError when either bound is exceeded.
    """
    o_tolerance = 2e-2 if dtype == torch.bfloat16 else 1e-2
    o_error = (actual_o.float().cpu() - expected_o.float()).abs().max().item()
    finite = torch.isfinite(expected_lse)
    got, want = actual_lse.float().cpu(), expected_lse.float()
    assert torch.equal(torch.isfinite(got), finite), "LSE finiteness pattern differs"
    assert torch.equal(got[~finite], want[~finite]), "non-finite LSE values differ"
    if finite.any():
        lse_error = ((got[finite] - want[finite]).abs() / want[finite].abs().clamp_min(0.1)).max().item()
    else:
        lse_error = 0.0
    assert math.isfinite(o_error) and o_error <= o_tolerance, f"O max-abs error {o_error} > {o_tolerance}"
    assert lse_error <= 1e-3, f"LSE relative error {lse_error} > 1e-3"
    return o_error, lse_error

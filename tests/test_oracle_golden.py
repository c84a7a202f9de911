"""Pin the CPU oracle against vectors produced by the reference's own CPU attention.

The fixtures come from ``tilecadence/bench_exchange.py:54-60`` (``_reference``) imported from the
reference tree by ``tests/golden/make_golden.py``.
"""
import importlib.util
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import attention as oracle

GOLDEN = Path(__file__).parent / "golden"


@pytest.fixture(scope="module")
def golden():
    spec = importlib.util.spec_from_file_location("make_golden", GOLDEN / "make_golden.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module, np.load(GOLDEN / "attention_golden.npz")


def compare(module, data, case, inputs, out, lse):
    assert bytes(module.digest(*inputs)) == bytes(data[f"{case}_inputs_sha256"]), "seeded inputs drifted"
    stride = module.STRIDES[case]
    np.testing.assert_allclose(out[:, ::stride].numpy(), data[f"{case}_o_rows"], rtol=1e-5, atol=2e-6)
    np.testing.assert_allclose(lse.numpy(), data[f"{case}_lse"], rtol=1e-5, atol=2e-6)
    checksum = np.array([out.double().sum().item(), out.double().abs().sum().item()])
    np.testing.assert_allclose(checksum, data[f"{case}_o_checksum"], rtol=1e-6)


def test_two_tile_noncausal_fp16(golden):
    module, data = golden
    q, k, v = module.golden_inputs("two_tile")
    out, lse = oracle.attention(q, k, v, causal=False)
    compare(module, data, "two_tile", (q, k, v), out, lse)


def test_causal_gqa_prefill_bf16(golden):
    module, data = golden
    q, k, v = module.golden_inputs("prefill")
    for row_block in (1024, 50):
        out, lse = oracle.attention(q, k, v, causal=True, row_block=row_block)
        compare(module, data, "prefill", (q, k, v), out, lse)


def test_decode_with_append(golden):
    module, data = golden
    kcache, vcache, q, knew, vnew, old = module.golden_inputs("decode")
    out, lse, kafter, vafter = oracle.decode_step(q, kcache, vcache, knew, vnew, old, append=True)
    compare(module, data, "decode", (kcache, vcache, q, knew, vnew), out, lse.transpose(1, 2).reshape(2, 8, 1))
    for b, length in enumerate(old.tolist()):
        assert torch.equal(kafter[b, length].view(torch.int16), knew[b, 0].view(torch.int16))
        assert torch.equal(vafter[b, length].view(torch.int16), vnew[b, 0].view(torch.int16))
        keep = torch.ones(200, dtype=torch.bool)
        keep[length] = False
        assert torch.equal(kafter[b, keep].view(torch.int16), kcache[b, keep].view(torch.int16))


def test_sharded_partials_merge_to_the_unsharded_result():
    """Split anywhere along the KV sequence, merge with the LSE combine: same O and LSE."""
    kcache, vcache, q, knew, vnew = oracle.seeded_normal(11, (2, 96, 2, 128), (2, 96, 2, 128), (2, 1, 8, 128),
                                                         (2, 1, 2, 128), (2, 1, 2, 128))
    old = torch.tensor([70, 3], dtype=torch.int32)
    want_o, want_lse, want_k, _ = oracle.decode_step(q, kcache, vcache, knew, vnew, old)
    parts_o, parts_lse, rows = [], [], []
    for start in (0, 32, 64):
        o, lse, kshard, _ = oracle.decode_step(q, kcache[:, start:start + 32], vcache[:, start:start + 32], knew, vnew,
                                               old, shard_start=start, partial=True)
        parts_o.append(o.reshape(16, 128))
        parts_lse.append(lse.reshape(16))
        rows.append(kshard)
    assert torch.equal(torch.cat(rows, dim=1).view(torch.int16), want_k.view(torch.int16))
    merged_o, merged_lse = oracle.combine(torch.stack(parts_o), torch.stack(parts_lse))
    torch.testing.assert_close(merged_o, want_o.reshape(16, 128), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(merged_lse, want_lse.reshape(16), rtol=1e-5, atol=1e-6)


def test_combine_handles_empty_parts():
    o = torch.randn(3, 4, 128)
    lse = torch.tensor([[0.5, float("-inf"), float("-inf"), 1.0],
                        [float("-inf"), float("-inf"), 2.0, 1.0],
                        [float("-inf"), float("-inf"), float("-inf"), 1.0]])
    o[1, 1] = float("nan")  # an unused part may hold anything
    merged, merged_lse = oracle.combine(o, lse)
    assert torch.equal(merged[0], o[0, 0]) and merged_lse[0] == 0.5
    assert torch.equal(merged[1], torch.zeros(128)) and merged_lse[1] == float("inf")
    assert torch.equal(merged[2], o[1, 2])
    torch.testing.assert_close(merged[3], o[:, 3].mean(dim=0))
    torch.testing.assert_close(merged_lse[3], torch.tensor(1.0 + np.log(3.0), dtype=torch.float32))


def test_indexed_caches_equal_the_gathered_contiguous_step():
    """Paged and batch-indexed decode in the oracle are the contiguous step on the gathered rows, and
    only the appended row of the owning page / slot changes."""
    batch, pages, page = 2, 7, 64
    kcache, vcache, q, knew, vnew = oracle.seeded_normal(
        5, (pages, page, 8, 128), (pages, page, 8, 128), (batch, 1, 32, 128), (batch, 1, 8, 128), (batch, 1, 8, 128))
    table = torch.tensor([[3, 0, 5], [6, 1, 2]], dtype=torch.int32)
    old = torch.tensor([130, 64], dtype=torch.int32)
    out, lse, k_after, v_after = oracle.decode_step_indexed(q, kcache, vcache, knew, vnew, old, block_table=table)
    gathered_k, gathered_v = kcache[table.long()].flatten(1, 2), vcache[table.long()].flatten(1, 2)
    want_o, want_lse, _, _ = oracle.decode_step(q, gathered_k, gathered_v, knew, vnew, old)
    assert torch.equal(out, want_o) and torch.equal(lse, want_lse)
    changed = (k_after != kcache).any(dim=(2, 3)).nonzero().tolist()
    assert changed == [[1, 0], [5, 2]]  # row 64 of sequence 1 -> page 1 row 0; row 130 of sequence 0 -> page 5 row 2
    assert torch.equal(k_after[5, 2], knew[0, 0]) and torch.equal(v_after[1, 0], vnew[1, 0])

    slots = torch.tensor([4, 1], dtype=torch.int32)
    old = torch.tensor([10, 63], dtype=torch.int32)
    out, lse, k_after, _ = oracle.decode_step_indexed(q, kcache, vcache, knew, vnew, old, cache_batch_idx=slots)
    want_o, want_lse, _, _ = oracle.decode_step(q, kcache[slots.long()], vcache[slots.long()], knew, vnew, old)
    assert torch.equal(out, want_o) and torch.equal(lse, want_lse)
    assert (k_after != kcache).any(dim=(2, 3)).nonzero().tolist() == [[1, 63], [4, 10]]
    with pytest.raises(ValueError):
        oracle.decode_step_indexed(q, kcache, vcache, knew, vnew, old)


def test_rotary_embedding_restatement():
    """rope_rotate is the published rotate-half form: identity at position 0, the textbook
    x*cos + rotate_half(x)*sin, a pure rotation of each (i, i+64) pair, and scores that depend only on
    the distance between the two positions."""
    cos, sin = oracle.rope_tables(512)
    assert cos.shape == (512, 64) and torch.all(cos[0] == 1) and torch.all(sin[0] == 0)
    assert abs(cos[1, 0].item() - 0.5403023) < 1e-6 and abs(sin[1, 0].item() - 0.8414710) < 1e-6  # angle 1 rad
    x, y = oracle.seeded_normal(12, (3, 1, 8, 128), (3, 1, 8, 128), dtype=torch.float32)
    position = torch.tensor([0, 17, 511])
    c, s = cos[position][:, None, None, :], sin[position][:, None, None, :]
    rotated = oracle.rope_rotate(x, c, s)
    assert torch.equal(rotated[0], x[0])
    rotate_half = torch.cat([-x[..., 64:], x[..., :64]], dim=-1)
    textbook = x * torch.cat([c, c], dim=-1) + rotate_half * torch.cat([s, s], dim=-1)
    assert torch.allclose(rotated, textbook, rtol=0, atol=1e-6)
    pair_norm = lambda t: t[..., :64] ** 2 + t[..., 64:] ** 2
    assert torch.allclose(pair_norm(rotated), pair_norm(x), rtol=1e-5, atol=1e-6)
    # <R_m x, R_n y> depends on m - n only
    a = (oracle.rope_rotate(x[:1], cos[40], sin[40]) * oracle.rope_rotate(y[:1], cos[33], sin[33])).sum(-1)
    b = (oracle.rope_rotate(x[:1], cos[107], sin[107]) * oracle.rope_rotate(y[:1], cos[100], sin[100])).sum(-1)
    assert torch.allclose(a, b, rtol=1e-4, atol=1e-3)
    # the fused step is the plain step on rotated, re-rounded inputs
    kcache, vcache, q, knew, vnew = oracle.seeded_normal(3, (2, 96, 8, 128), (2, 96, 8, 128), (2, 1, 32, 128),
                                                         (2, 1, 8, 128), (2, 1, 8, 128))
    old = torch.tensor([40, 95], dtype=torch.int32)
    got = oracle.decode_step_rope(q, kcache, vcache, knew, vnew, old, cos, sin)
    pc, ps = cos[old.long()][:, None, None, :], sin[old.long()][:, None, None, :]
    want = oracle.decode_step(oracle.rope_rotate(q, pc, ps), kcache, vcache, oracle.rope_rotate(knew, pc, ps), vnew, old)
    assert all(torch.equal(g, w) for g, w in zip(got, want))
    assert torch.equal(got[2][0, 40], oracle.rope_rotate(knew, pc, ps)[0, 0]) and got[2].dtype == torch.bfloat16


def test_projection_step_restatement():
    """project_qkv_rope = matmul, then exactly the norm and RoPE functions above, head by head."""
    x, w, qn, kn = oracle.seeded_normal(8, (3, 256), (48 * 128, 256), (128,), (128,), dtype=torch.float32)
    x, w = x.to(torch.bfloat16), (w / 16).to(torch.bfloat16)
    qn, kn = (1 + 0.1 * qn).to(torch.bfloat16), (1 + 0.1 * kn).to(torch.bfloat16)
    cos, sin = oracle.rope_tables(64)
    positions = torch.tensor([0, 5, 63], dtype=torch.int32)
    q, k, v = oracle.project_qkv_rope(x, w, positions, 32, 8, qn, kn, cos, sin)
    assert q.shape == (3, 1, 32, 128) and k.shape == (3, 1, 8, 128) and v.shape == (3, 1, 8, 128)
    y = (x.float() @ w.float().T).view(3, 48, 128)
    assert torch.equal(v[:, 0], y[:, 40:].to(torch.bfloat16))
    head = y[1, 33]  # a k head of token 1
    normed = ((head * torch.rsqrt(head.pow(2).mean() + 1e-6)).to(torch.bfloat16).float() * kn.float()).to(torch.bfloat16)
    assert torch.equal(k[1, 0, 1], oracle.rope_rotate(normed, cos[5], sin[5]))
    plain = oracle.project_qkv_rope(x, w, None, 32, 8)
    assert torch.equal(plain[0][:, 0], y[:, :32].to(torch.bfloat16))
    assert torch.equal(q[0], oracle.project_qkv_rope(x, w, positions, 32, 8, qn, kn)[0][0])  # position 0: no rotation

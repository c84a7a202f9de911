"""Parity of the tcgen05 causal GQA prefill kernel with the CPU oracle, through the C ABI.

Tolerances: O max-abs error <= 2e-2 (BF16), LSE <= 1e-3 relative. Follows the reference's prefill
verification (``tilecadence/bench_operator.py:29-43``): both mappings run on the same inputs and
must agree bit for bit.
"""
import pytest
import torch

from oracle import attention as oracle
from tilecadence_b200 import cuda_runtime

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(library):
    return cuda_runtime.ops_for(library, "prefill")


def run_prefill(ops, device, q, k, v, mapping=1, scale=128 ** -0.5):
    dq, dk, dv = q.to(device), k.to(device), v.to(device)
    out = torch.full(dq.shape, float("nan"), device=device, dtype=torch.bfloat16)
    lse = torch.full((q.size(0), q.size(2), q.size(1)), float("nan"), device=device, dtype=torch.float32)
    empty = torch.empty(0, device=device, dtype=torch.float32)
    assert ops.workspace_spec(dq, dk, dv, 0, mapping, True) == [1, 0, 0]
    ops.forward_out(dq, dk, dv, out, lse, empty, empty, 0, mapping, scale, True)
    torch.cuda.synchronize()
    assert ops.library.device_status(device.index) == 0
    return out.cpu(), lse.cpu()


def bits(tensor, integer=torch.int16):
    return tensor.contiguous().view(integer)


@pytest.mark.parametrize("batch,tokens", [(1, 128), (1, 256), (1, 193), (4, 384), (1, 1537), (1, 2048)])
def test_prefill_matches_oracle(ops, gpu_device, batch, tokens):
    q, k, v = oracle.seeded_normal(2000 + tokens, (batch, tokens, 32, 128), (batch, tokens, 8, 128),
                                   (batch, tokens, 8, 128))
    want_o, want_lse = oracle.attention(q, k, v, causal=True)
    got_o, got_lse = run_prefill(ops, gpu_device, q, k, v)
    oracle.check_outputs(got_o, got_lse, want_o, want_lse)


def test_mappings_agree_bitwise(ops, gpu_device):
    q, k, v = oracle.seeded_normal(5, (1, 640, 32, 128), (1, 640, 8, 128), (1, 640, 8, 128))
    o0, l0 = run_prefill(ops, gpu_device, q, k, v, mapping=0)
    o1, l1 = run_prefill(ops, gpu_device, q, k, v, mapping=1)
    assert torch.isfinite(o1.float()).all() and torch.isfinite(l1).all()
    assert torch.equal(bits(o0), bits(o1)) and torch.equal(bits(l0, torch.int32), bits(l1, torch.int32))


def test_strided_inputs_and_custom_scale(ops, gpu_device):
    """Q/K/V views into a packed QKV projection (row stride 48*128) and a non-default scale."""
    (packed,) = oracle.seeded_normal(6, (1, 512, 48, 128))
    q, k, v = packed[:, :, :32], packed[:, :, 32:40], packed[:, :, 40:]
    want_o, want_lse = oracle.attention(q, k, v, causal=True, scale=0.05)
    device_packed = packed.to(gpu_device)
    dq, dk, dv = device_packed[:, :, :32], device_packed[:, :, 32:40], device_packed[:, :, 40:]
    out = torch.empty((1, 512, 32, 128), device=gpu_device, dtype=torch.bfloat16)
    lse = torch.empty((1, 32, 512), device=gpu_device, dtype=torch.float32)
    empty = torch.empty(0, device=gpu_device, dtype=torch.float32)
    ops.forward_out(dq, dk, dv, out, lse, empty, empty, 0, 1, 0.05, True)
    torch.cuda.synchronize()
    oracle.check_outputs(out.cpu(), lse.cpu(), want_o, want_lse)


@pytest.mark.parametrize("scale", [1.0, 0.35])
def test_sharp_softmax_exercises_the_rescale_path(ops, gpu_device, scale):
    """With a large scale the running row maximum jumps by far more than 2^8 between tiles, so the
    gated O rescale (TMEM read-modify-write) runs many times; with the default scale it almost never does."""
    q, k, v = oracle.seeded_normal(8, (1, 1024, 32, 128), (1, 1024, 8, 128), (1, 1024, 8, 128))
    want_o, want_lse = oracle.attention(q, k, v, causal=True, scale=scale)
    got_o, got_lse = run_prefill(ops, gpu_device, q, k, v, scale=scale)
    oracle.check_outputs(got_o, got_lse, want_o, want_lse)


def test_head_group_shard(library, gpu_device):
    """A KV-head-group shard (8 query heads over 2 KV heads) equals the same heads of the full run."""
    q, k, v = oracle.seeded_normal(7, (1, 256, 32, 128), (1, 256, 8, 128), (1, 256, 8, 128))
    want_o, want_lse = oracle.attention(q, k, v, causal=True)
    shard_ops = cuda_runtime.ops_for(library, "prefill", q_heads=8)
    got_o, got_lse = run_prefill(shard_ops, gpu_device, q[:, :, 8:16].contiguous(), k[:, :, 2:4].contiguous(),
                                 v[:, :, 2:4].contiguous())
    oracle.check_outputs(got_o, got_lse, want_o[:, :, 8:16], want_lse[:, 8:16])


def run_key_split(ops, device, q, k, v, key_splits, mapping=1, scale=128 ** -0.5, repeats=1):
    dq, dk, dv = q.to(device), k.to(device), v.to(device)
    out = torch.full(dq.shape, float("nan"), device=device, dtype=torch.bfloat16)
    lse = torch.full((q.size(0), q.size(2), q.size(1)), float("nan"), device=device, dtype=torch.float32)
    # The workspace starts as garbage: the call itself has to clear what it relies on.
    workspace = torch.full((ops.key_split_workspace_bytes(dq),), 0xA5, device=device, dtype=torch.uint8)
    for _ in range(repeats):
        used = ops.key_split_forward_out(dq, dk, dv, out, lse, workspace, mapping, scale, key_splits)
    torch.cuda.synchronize()
    assert ops.library.device_status(device.index) == 0
    return out.cpu(), lse.cpu(), used


@pytest.mark.parametrize("heads,batch,tokens", [(4, 1, 128), (4, 1, 256), (8, 1, 193), (4, 4, 384), (4, 1, 1537),
                                                (32, 1, 1024)])
def test_two_ctas_per_query_tile_match_the_oracle(library, gpu_device, heads, batch, tokens):
    """Key-split prefill: one, two, three (uneven halves), ragged and many key tiles per query tile."""
    shard_ops = cuda_runtime.ops_for(library, "prefill", q_heads=heads)
    q, k, v = oracle.seeded_normal(4000 + tokens, (batch, tokens, heads, 128), (batch, tokens, heads // 4, 128),
                                   (batch, tokens, heads // 4, 128))
    want_o, want_lse = oracle.attention(q, k, v, causal=True)
    got_o, got_lse, used = run_key_split(shard_ops, gpu_device, q, k, v, key_splits=2, repeats=2)
    assert used == 2
    oracle.check_outputs(got_o, got_lse, want_o, want_lse)


def test_key_split_of_one_is_the_plain_kernel_and_mappings_agree(library, gpu_device):
    shard_ops = cuda_runtime.ops_for(library, "prefill", q_heads=8)
    q, k, v = oracle.seeded_normal(11, (1, 896, 8, 128), (1, 896, 2, 128), (1, 896, 2, 128))
    plain_o, plain_lse = run_prefill(shard_ops, gpu_device, q, k, v)
    one_o, one_lse, used = run_key_split(shard_ops, gpu_device, q, k, v, key_splits=1)
    assert used == 1
    assert torch.equal(bits(plain_o), bits(one_o)) and torch.equal(bits(plain_lse, torch.int32), bits(one_lse, torch.int32))
    two_o, two_lse, _ = run_key_split(shard_ops, gpu_device, q, k, v, key_splits=2)
    oracle.check_outputs(two_o, two_lse, plain_o.float(), plain_lse)
    # Which CTA of a pair finishes second is a race, and the merge is not symmetric in rounding, so two
    # runs are compared to tolerance; the two staging mappings of one run order agree to tolerance too.
    other_o, other_lse, _ = run_key_split(shard_ops, gpu_device, q, k, v, key_splits=2, mapping=0)
    oracle.check_outputs(other_o, other_lse, two_o.float(), two_lse)


def test_key_split_is_chosen_for_a_head_group_shard_of_config2(library, gpu_device):
    """One KV head's shard of config 2 (what each of 8 GPUs holds): 128 query-tile CTAs cannot fill 148 SMs,
    so the automatic choice is two CTAs per tile; the full 32-head problem keeps one."""
    tokens = 8192
    q, k, v = oracle.seeded_normal(1, (1, tokens, 32, 128), (1, tokens, 8, 128), (1, tokens, 8, 128))
    shard_ops = cuda_runtime.ops_for(library, "prefill", q_heads=4)
    sq, sk, sv = q[:, :, 4:8].contiguous(), k[:, :, 1:2].contiguous(), v[:, :, 1:2].contiguous()
    got_o, got_lse, used = run_key_split(shard_ops, gpu_device, sq, sk, sv, key_splits=0)
    assert used == 2
    want_o, want_lse = oracle.attention(sq, sk, sv, causal=True, row_block=512)
    oracle.check_outputs(got_o, got_lse, want_o, want_lse)
    full_ops = cuda_runtime.ops_for(library, "prefill")
    dq, dk, dv = (t.to(gpu_device) for t in (q, k, v))
    out, lse = torch.empty_like(dq), torch.empty((1, 32, tokens), device=gpu_device)
    workspace = torch.empty(full_ops.key_split_workspace_bytes(dq), device=gpu_device, dtype=torch.uint8)
    assert full_ops.key_split_forward_out(dq, dk, dv, out, lse, workspace, 1, 128 ** -0.5, 0) == 1


def test_config2_full_size(ops, gpu_device):
    """BASELINE config 2: batch 1, 8192 tokens, 32 query / 8 KV heads, seed 1."""
    q, k, v = oracle.seeded_normal(1, (1, 8192, 32, 128), (1, 8192, 8, 128), (1, 8192, 8, 128))
    got_o, got_lse = run_prefill(ops, gpu_device, q, k, v)
    torch.set_num_threads(max(1, torch.get_num_threads()))
    want_o, want_lse = oracle.attention(q, k, v, causal=True, row_block=512)
    oracle.check_outputs(got_o, got_lse, want_o, want_lse)


def test_full_size_properties_causality_and_linearity_in_v(ops, gpu_device):
    """Two properties that need no oracle pass, at config-2 size. Causality: replacing every key and value row
    from 5000 on changes no bit of the outputs of the rows before it (a query tile's CTA runs the same
    instructions on the same data whatever else is in the launch). Linearity: the probabilities do not
    depend on V, so O(V1 + V2) = O(V1) + O(V2) up to the BF16 roundings of the three outputs."""
    tokens, cut = 8192, 5000
    q, k, v = oracle.seeded_normal(21, (1, tokens, 32, 128), (1, tokens, 8, 128), (1, tokens, 8, 128))
    base_o, base_lse = run_prefill(ops, gpu_device, q, k, v)
    k2, v2 = k.clone(), v.clone()
    other_k, other_v = oracle.seeded_normal(22, (1, tokens - cut, 8, 128), (1, tokens - cut, 8, 128))
    k2[:, cut:], v2[:, cut:] = other_k, other_v
    changed_o, changed_lse = run_prefill(ops, gpu_device, q, k2, v2)
    assert torch.equal(bits(base_o[:, :cut]), bits(changed_o[:, :cut]))
    assert torch.equal(bits(base_lse[:, :, :cut], torch.int32), bits(changed_lse[:, :, :cut], torch.int32))
    assert not torch.equal(bits(base_o[:, cut:]), bits(changed_o[:, cut:]))
    _, _, w = oracle.seeded_normal(23, (1, 1, 1, 1), (1, 1, 1, 1), (1, tokens, 8, 128))
    total = (v.float() + w.float()).to(torch.bfloat16)       # what the kernel sees as V1 + V2 ...
    second = (total.float() - v.float()).to(torch.bfloat16)  # ... and the V2 that goes with it
    sum_o, sum_lse = run_prefill(ops, gpu_device, q, k, total)
    second_o, second_lse = run_prefill(ops, gpu_device, q, k, second)
    assert torch.equal(bits(sum_lse, torch.int32), bits(base_lse, torch.int32))
    assert torch.equal(bits(second_lse, torch.int32), bits(base_lse, torch.int32))
    error = (sum_o.float() - (base_o.float() + second_o.float())).abs().max().item()
    assert error <= 2 ** -6 * max(1.0, sum_o.float().abs().max().item())


def test_long_sequence_rows_against_oracle(ops, gpu_device):
    """32768 tokens, batch 1: every row's LSE is finite and a sample of rows matches the oracle."""
    tokens = 32768
    q, k, v = oracle.seeded_normal(2, (1, tokens, 32, 128), (1, tokens, 8, 128), (1, tokens, 8, 128))
    got_o, got_lse = run_prefill(ops, gpu_device, q, k, v)
    assert torch.isfinite(got_lse).all() and torch.isfinite(got_o.float()).all()
    for r0 in (0, 12345, tokens - 64):
        rows = slice(r0, r0 + 64)
        for g in (0, 5):
            qh = q[0, rows, g * 4:(g + 1) * 4].float().permute(1, 0, 2)
            scores = (qh @ k[0, :r0 + 64, g].float().T) * 128 ** -0.5
            cols = torch.arange(r0 + 64)[None, :]
            scores.masked_fill_(cols > torch.arange(r0, r0 + 64)[:, None], float("-inf"))
            want_lse = scores.logsumexp(-1)
            want_o = (scores.softmax(-1) @ v[0, :r0 + 64, g].float()).permute(1, 0, 2)
            oracle.check_outputs(got_o[0, rows, g * 4:(g + 1) * 4], got_lse[0, g * 4:(g + 1) * 4, rows], want_o, want_lse)


@pytest.mark.parametrize("tokens", [8193, 12289, 4225])
def test_ragged_long_sequences(ops, gpu_device, tokens):
    """Lengths the reference studies that are no multiple of the tile (8193, 12289) and one just above the
    switch between the two schedules: the last query tile holds a single row or 65 rows. Sampled row blocks,
    the ragged end among them, against the oracle; nothing is written past the last row."""
    q, k, v = oracle.seeded_normal(tokens, (1, tokens, 32, 128), (1, tokens, 8, 128), (1, tokens, 8, 128))
    got_o, got_lse = run_prefill(ops, gpu_device, q, k, v)
    assert torch.isfinite(got_lse).all() and torch.isfinite(got_o.float()).all()
    for r0, count in ((0, 64), (tokens // 2 - 7, 64), (tokens - 65, 65)):
        rows = slice(r0, r0 + count)
        for g in (1, 7):
            qh = q[0, rows, g * 4:(g + 1) * 4].float().permute(1, 0, 2)
            scores = (qh @ k[0, :r0 + count, g].float().T) * 128 ** -0.5
            cols = torch.arange(r0 + count)[None, :]
            scores.masked_fill_(cols > torch.arange(r0, r0 + count)[:, None], float("-inf"))
            want_lse = scores.logsumexp(-1)
            want_o = (scores.softmax(-1) @ v[0, :r0 + count, g].float()).permute(1, 0, 2)
            oracle.check_outputs(got_o[0, rows, g * 4:(g + 1) * 4], got_lse[0, g * 4:(g + 1) * 4, rows], want_o, want_lse)


def test_batch_four_is_four_independent_sequences(ops, gpu_device):
    """Config-3 shape B4 x 8192: every sequence of the batch gives the bits of the same sequence run alone,
    and a sample of rows of the last sequence matches the oracle."""
    tokens = 8192
    q, k, v = oracle.seeded_normal(2, (4, tokens, 32, 128), (4, tokens, 8, 128), (4, tokens, 8, 128))
    got_o, got_lse = run_prefill(ops, gpu_device, q, k, v)
    for b in (0, 3):
        alone_o, alone_lse = run_prefill(ops, gpu_device, q[b:b + 1], k[b:b + 1], v[b:b + 1])
        assert torch.equal(bits(alone_o[0]), bits(got_o[b]))
        assert torch.equal(alone_lse[0].view(torch.int32), got_lse[b].view(torch.int32))
    r0, g = 5000, 6
    rows = slice(r0, r0 + 64)
    qh = q[3, rows, g * 4:(g + 1) * 4].float().permute(1, 0, 2)
    scores = (qh @ k[3, :r0 + 64, g].float().T) * 128 ** -0.5
    scores.masked_fill_(torch.arange(r0 + 64)[None, :] > torch.arange(r0, r0 + 64)[:, None], float("-inf"))
    want_o = (scores.softmax(-1) @ v[3, :r0 + 64, g].float()).permute(1, 0, 2)
    oracle.check_outputs(got_o[3, rows, g * 4:(g + 1) * 4], got_lse[3, g * 4:(g + 1) * 4, rows], want_o,
                         scores.logsumexp(-1))


def test_argument_checks(ops, gpu_device):
    q, k, v = (t.to(gpu_device) for t in oracle.seeded_normal(1, (1, 128, 32, 128), (1, 128, 8, 128), (1, 128, 8, 128)))
    out, lse = torch.empty_like(q), torch.empty((1, 32, 128), device=gpu_device)
    empty = torch.empty(0, device=gpu_device)
    with pytest.raises(RuntimeError, match="causal"):
        ops.forward_out(q, k, v, out, lse, empty, empty, 0, 1, 0.1, False)
    with pytest.raises(RuntimeError, match="num_splits=0"):
        ops.workspace_spec(q, k, v, 2, 1, True)
    with pytest.raises(RuntimeError, match="scale"):
        ops.forward_out(q, k, v, out, lse, empty, empty, 0, 1, float("nan"), True)
    with pytest.raises(RuntimeError, match="aliases"):
        ops.forward_out(q, k, v, q, lse, empty, empty, 0, 1, 0.1, True)
    with pytest.raises(RuntimeError, match="batch 1 or 4"):
        ops.workspace_spec(q.expand(2, -1, -1, -1).contiguous(), k.expand(2, -1, -1, -1).contiguous(),
                           v.expand(2, -1, -1, -1).contiguous(), 0, 1, True)
    resources = ops.resources(q, k, v, 0, 1, True)
    assert len(resources) == 46 and resources[12] == 384 and resources[19] == 1

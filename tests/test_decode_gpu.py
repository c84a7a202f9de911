"""Parity of the fused split-KV decode kernel with the CPU oracle, through the C ABI.

Tolerances (the acceptance bar of this path): O max-abs error <= 2e-2 (BF16), LSE <= 1e-3
relative, cache appends and untouched rows bit-exact. The checks follow the reference's own
decode verification (``tilecadence/bench_operator.py:46-78``): two consecutive steps, history and
both appended rows compared as raw 16-bit words, and bitwise equality between the two mappings.
"""
import pytest
import torch

from oracle import attention as oracle
from tilecadence_b200 import cuda_runtime

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(library):
    return cuda_runtime.ops_for(library, "decode")


def run_step(ops, device, q, kcache, vcache, knew, vnew, old, mapping=1, num_splits=0, append=True):
    """Run one step on device copies; returns (O, LSE, kcache_after, vcache_after) on the host."""
    dq, dk, dv, dkn, dvn = (t.to(device) for t in (q, kcache, vcache, knew, vnew))
    dold = old.to(device=device, dtype=torch.int32)
    out = torch.full_like(dq, float("nan"))
    lse = torch.full((q.size(0), q.size(2), 1), float("nan"), device=device, dtype=torch.float32)
    spec = ops.workspace_spec(dq, dk, dold, num_splits, mapping, append)
    ws_o = torch.full((spec[1],), float("nan"), device=device, dtype=torch.float32)
    ws_lse = torch.full((spec[2],), float("nan"), device=device, dtype=torch.float32)
    ops.forward_out(dq, dk, dv, dkn, dvn, dold, out, lse, ws_o, ws_lse, num_splits, mapping, append)
    torch.cuda.synchronize()
    assert ops.library.device_status(device.index) == 0
    return out.cpu(), lse.cpu(), dk.cpu(), dv.cpu(), spec


def make_case(seed, batch, capacity, kv_heads=8, fill=None):
    kcache, vcache, q, knew, vnew = oracle.seeded_normal(
        seed, (batch, capacity, kv_heads, 128), (batch, capacity, kv_heads, 128), (batch, 1, kv_heads * 4, 128),
        (batch, 1, kv_heads, 128), (batch, 1, kv_heads, 128))
    if fill is not None:  # rows past the valid prefix hold NaN bit patterns: they must never matter
        for b, length in enumerate(fill):
            kcache[b, length:] = float("nan")
            vcache[b, length:] = float("nan")
    return q, kcache, vcache, knew, vnew


def bits(tensor):
    return tensor.contiguous().view(torch.int16)


@pytest.mark.parametrize("batch,capacity,lengths", [
    (1, 200, [130]),
    (2, 200, [130, 7]),
    (1, 64, [0]),                 # the appended row is the only visible key
    (1, 65, [64]),                # append lands in the last, one-row tile at the end of capacity
    (4, 1024, [1023, 0, 511, 64]),  # ragged batch, one sequence filling the cache
    (1, 4096, [2500]),
    (1, 16384, [8193]),           # lengths the reference studies: one row past a tile boundary
    (2, 16384, [12289, 192]),
])
def test_decode_matches_oracle(ops, gpu_device, batch, capacity, lengths):
    q, kcache, vcache, knew, vnew = make_case(100 + capacity, batch, capacity, fill=lengths)
    old = torch.tensor(lengths, dtype=torch.int32)
    want_o, want_lse, want_k, want_v = oracle.decode_step(q, kcache, vcache, knew, vnew, old)
    got_o, got_lse, got_k, got_v, _ = run_step(ops, gpu_device, q, kcache, vcache, knew, vnew, old)
    oracle.check_outputs(got_o, got_lse, want_o, want_lse)
    assert torch.equal(bits(got_k), bits(want_k)) and torch.equal(bits(got_v), bits(want_v))


def test_two_steps_like_the_reference_harness(ops, gpu_device):
    """Config 4 geometry at reduced capacity: prefix, then two appended tokens (bench_operator.py:46-78)."""
    batch, length = 1, 1000
    prefix_k, prefix_v = oracle.seeded_normal(3, (batch, length, 8, 128), (batch, length, 8, 128))
    steps = [oracle.seeded_normal(30 + s, (batch, 1, 32, 128), (batch, 1, 8, 128), (batch, 1, 8, 128)) for s in range(2)]
    results = []
    for mapping in (0, 1):
        kcache = torch.zeros((batch, length + 2, 8, 128), dtype=torch.bfloat16)
        vcache = torch.zeros_like(kcache)
        kcache[:, :length], vcache[:, :length] = prefix_k, prefix_v
        outputs = []
        for step, (q, knew, vnew) in enumerate(steps):
            old = torch.full((batch,), length + step, dtype=torch.int32)
            want_o, want_lse, want_k, want_v = oracle.decode_step(q, kcache, vcache, knew, vnew, old)
            got_o, got_lse, kcache, vcache, _ = run_step(ops, gpu_device, q, kcache, vcache, knew, vnew, old, mapping)
            oracle.check_outputs(got_o, got_lse, want_o, want_lse)
            assert torch.equal(bits(kcache), bits(want_k)) and torch.equal(bits(vcache), bits(want_v))
            outputs.append((got_o, got_lse))
        for idx, (cache, prefix) in enumerate(((kcache, prefix_k), (vcache, prefix_v))):
            assert torch.equal(bits(cache[:, :length]), bits(prefix))
            assert torch.equal(bits(cache[:, length:length + 1]), bits(steps[0][idx + 1]))
            assert torch.equal(bits(cache[:, length + 1:length + 2]), bits(steps[1][idx + 1]))
        results.append(outputs)
    for (o0, l0), (o1, l1) in zip(*results):  # the two mappings agree bit for bit
        assert torch.equal(bits(o0), bits(o1)) and torch.equal(l0.view(torch.int32), l1.view(torch.int32))


@pytest.mark.parametrize("num_splits", [1, 2, 5, 37, 128])
def test_split_counts_agree(ops, gpu_device, num_splits):
    q, kcache, vcache, knew, vnew = make_case(7, 2, 3000, fill=[2999, 100])
    old = torch.tensor([2999, 100], dtype=torch.int32)
    want_o, want_lse, want_k, want_v = oracle.decode_step(q, kcache, vcache, knew, vnew, old)
    got_o, got_lse, got_k, got_v, spec = run_step(ops, gpu_device, q, kcache, vcache, knew, vnew, old,
                                                  num_splits=num_splits)
    assert spec[0] == num_splits and spec[1] == (0 if num_splits == 1 else num_splits * 2 * 32 * 128)
    oracle.check_outputs(got_o, got_lse, want_o, want_lse)
    assert torch.equal(bits(got_k), bits(want_k)) and torch.equal(bits(got_v), bits(want_v))


def test_without_append_the_cache_is_untouched(ops, gpu_device):
    q, kcache, vcache, knew, vnew = make_case(8, 2, 300, fill=[300, 0])
    old = torch.tensor([300, 0], dtype=torch.int32)  # second sequence sees no key at all
    want_o, want_lse, _, _ = oracle.decode_step(q, kcache, vcache, knew, vnew, old, append=False)
    got_o, got_lse, got_k, got_v, _ = run_step(ops, gpu_device, q, kcache, vcache, knew, vnew, old, append=False)
    oracle.check_outputs(got_o, got_lse, want_o, want_lse)
    assert torch.isinf(got_lse[1]).all() and (got_lse[1] > 0).all() and (got_o[1] == 0).all()
    assert torch.equal(bits(got_k), bits(kcache)) and torch.equal(bits(got_v), bits(vcache))


def test_config4_full_size(ops, gpu_device):
    """BASELINE config 4: capacity 32768, 8192 valid tokens, seed 3, two appended tokens."""
    capacity, length = 32768, 8192
    kcache = torch.zeros((1, capacity, 8, 128), dtype=torch.bfloat16)
    vcache = torch.zeros_like(kcache)
    generator = torch.Generator().manual_seed(3)
    kcache[:, :length] = torch.randn((1, length, 8, 128), generator=generator).to(torch.bfloat16)
    vcache[:, :length] = torch.randn((1, length, 8, 128), generator=generator).to(torch.bfloat16)
    for step in range(2):
        q, knew, vnew = (torch.randn(shape, generator=generator).to(torch.bfloat16)
                         for shape in ((1, 1, 32, 128), (1, 1, 8, 128), (1, 1, 8, 128)))
        old = torch.tensor([length + step], dtype=torch.int32)
        want_o, want_lse, want_k, want_v = oracle.decode_step(q, kcache, vcache, knew, vnew, old)
        got_o, got_lse, kcache, vcache, _ = run_step(ops, gpu_device, q, kcache, vcache, knew, vnew, old)
        oracle.check_outputs(got_o, got_lse, want_o, want_lse)
        assert torch.equal(bits(kcache), bits(want_k)) and torch.equal(bits(vcache), bits(want_v))
    assert not kcache[:, length + 2:].any() and not vcache[:, length + 2:].any()


def test_config5_full_size(ops, gpu_device):
    """BASELINE config 5 on one GPU: batch 4, 32768 rows attended (old_len 32767, the new row lands in the
    last cache row), seed 4. Checked against the oracle, and against eight KV-sequence shards of the same
    caches merged by the combine kernel (the multi-GPU decomposition on one device)."""
    batch, capacity, shards = 4, 32768, 8
    generator = torch.Generator().manual_seed(4)
    kcache = torch.randn((batch, capacity, 8, 128), generator=generator).to(torch.bfloat16)
    vcache = torch.randn((batch, capacity, 8, 128), generator=generator).to(torch.bfloat16)
    q, knew, vnew = (torch.randn(shape, generator=generator).to(torch.bfloat16)
                     for shape in ((batch, 1, 32, 128), (batch, 1, 8, 128), (batch, 1, 8, 128)))
    old = torch.full((batch,), capacity - 1, dtype=torch.int32)
    want_o, want_lse, want_k, want_v = oracle.decode_step(q, kcache, vcache, knew, vnew, old)
    got_o, got_lse, got_k, got_v, _ = run_step(ops, gpu_device, q, kcache, vcache, knew, vnew, old)
    oracle.check_outputs(got_o, got_lse, want_o, want_lse)
    assert torch.equal(bits(got_k), bits(want_k)) and torch.equal(bits(got_v), bits(want_v))
    del got_k, got_v, want_k, want_v
    device = gpu_device
    dq, dkn, dvn, dold = q.to(device), knew.to(device), vnew.to(device), old.to(device)
    part_o = torch.empty((shards, batch * 32, 128), device=device, dtype=torch.float32)
    part_lse = torch.empty((shards, batch * 32), device=device, dtype=torch.float32)
    length = capacity // shards
    for s in range(shards):
        dk = kcache[:, s * length:(s + 1) * length].contiguous().to(device)
        dv = vcache[:, s * length:(s + 1) * length].contiguous().to(device)
        spec = ops.workspace_spec(dq, dk, dold, 0, 1, True)
        ws = [torch.empty(n, device=device, dtype=torch.float32) for n in spec[1:3]]
        ops.partial_out(dq, dk, dv, dkn, dvn, dold, part_o[s], part_lse[s], *ws, 0, 1, True, s * length)
    out = torch.empty((batch, 1, 32, 128), device=device, dtype=torch.bfloat16)
    lse = torch.empty((batch, 32, 1), device=device, dtype=torch.float32)
    ops.combine_partials(part_o, part_lse, out, lse)
    torch.cuda.synchronize()
    assert ops.library.device_status(device.index) == 0
    oracle.check_outputs(out.cpu(), lse.cpu(), want_o, want_lse)
    assert (out.cpu().float() - got_o.float()).abs().max().item() <= 2e-2


def test_full_size_properties_key_order_and_repeatability(ops, gpu_device):
    """Two properties at config-5 size that need no oracle pass. A step repeated on a copy of the same cache
    gives the same bits (no run-to-run race in the split merge). Attention does not depend on the order of
    the cached keys: the same rows in reversed order (values reversed with them) give the same O and LSE up
    to rounding, although every split then sees other rows."""
    batch, capacity, length = 4, 32768, 32767
    q, kcache, vcache, knew, vnew = make_case(31, batch, capacity)
    old = torch.full((batch,), length, dtype=torch.int32)
    first_o, first_lse, k_after, _, _ = run_step(ops, gpu_device, q, kcache, vcache, knew, vnew, old)
    again_o, again_lse, _, _, _ = run_step(ops, gpu_device, q, kcache, vcache, knew, vnew, old)
    assert torch.equal(bits(first_o), bits(again_o)) and torch.equal(first_lse.view(torch.int32), again_lse.view(torch.int32))
    assert torch.equal(bits(k_after[:, length]), bits(knew[:, 0]))
    reversed_k, reversed_v = kcache.clone(), vcache.clone()
    reversed_k[:, :length] = kcache[:, :length].flip(1)
    reversed_v[:, :length] = vcache[:, :length].flip(1)
    other_o, other_lse, _, _, _ = run_step(ops, gpu_device, q, reversed_k, reversed_v, knew, vnew, old)
    assert (other_o.float() - first_o.float()).abs().max().item() <= 2 ** -8
    assert torch.allclose(other_lse, first_lse, rtol=1e-5, atol=1e-5)


def test_sharded_partials_and_combine(ops, gpu_device):
    """KV-sequence shards produce partials whose LSE-weighted merge equals the unsharded step."""
    batch, capacity, shards = 4, 2048, 4
    q, kcache, vcache, knew, vnew = make_case(9, batch, capacity)
    old = torch.tensor([2047, 5, 1024, 600], dtype=torch.int32)
    want_o, want_lse, want_k, want_v = oracle.decode_step(q, kcache, vcache, knew, vnew, old)
    device = gpu_device
    dq, dkn, dvn, dold = q.to(device), knew.to(device), vnew.to(device), old.to(device)
    part_o = torch.empty((shards, batch * 32, 128), device=device, dtype=torch.float32)
    part_lse = torch.empty((shards, batch * 32), device=device, dtype=torch.float32)
    shard_len = capacity // shards
    caches = []
    for s in range(shards):
        dk = kcache[:, s * shard_len:(s + 1) * shard_len].contiguous().to(device)
        dv = vcache[:, s * shard_len:(s + 1) * shard_len].contiguous().to(device)
        spec = ops.workspace_spec(dq, dk, dold, 0, 1, True)
        ws_o = torch.empty((spec[1],), device=device, dtype=torch.float32)
        ws_lse = torch.empty((spec[2],), device=device, dtype=torch.float32)
        ops.partial_out(dq, dk, dv, dkn, dvn, dold, part_o[s], part_lse[s], ws_o, ws_lse, 0, 1, True, s * shard_len)
        caches.append((dk, dv))
    out = torch.empty((batch, 1, 32, 128), device=device, dtype=torch.bfloat16)
    lse = torch.empty((batch, 32, 1), device=device, dtype=torch.float32)
    ops.combine_partials(part_o, part_lse, out, lse)
    torch.cuda.synchronize()
    assert ops.library.device_status(device.index) == 0
    oracle.check_outputs(out.cpu(), lse.cpu(), want_o, want_lse)
    assert torch.equal(bits(torch.cat([k.cpu() for k, _ in caches], dim=1)), bits(want_k))
    assert torch.equal(bits(torch.cat([v.cpu() for _, v in caches], dim=1)), bits(want_v))
    # a shard that holds no visible key reports -inf and contributes nothing
    assert torch.isinf(part_lse[3].view(batch, 32)[1]).all()


def run_indexed(ops, device, q, kcache, vcache, knew, vnew, old, capacity, num_splits=0, **index):
    dq, dk, dv, dkn, dvn = (t.to(device) for t in (q, kcache, vcache, knew, vnew))
    dold = old.to(device)
    out = torch.full_like(dq, float("nan"))
    lse = torch.full((q.size(0), 32, 1), float("nan"), device=device, dtype=torch.float32)
    spec = ops.indexed_workspace_spec(q.size(0), capacity, 8, device.index, num_splits)
    ws = [torch.full((n,), float("nan"), device=device, dtype=torch.float32) for n in spec[1:3]]
    ops.indexed_forward_out(dq, dk, dv, dkn, dvn, dold, out, lse, *ws, num_splits, 1, True,
                            **{name: value.to(device) for name, value in index.items()})
    torch.cuda.synchronize()
    assert ops.library.device_status(device.index) == 0
    return out.cpu(), lse.cpu(), dk.cpu(), dv.cpu()


@pytest.mark.parametrize("page,pages_per_seq,lengths,num_splits", [
    (64, 5, [130, 64, 0], 0),
    (128, 8, [1023, 517, 128], 0),
    (256, 40, [10239, 4097, 255], 0),
    (64, 160, [10000, 9000, 8000], 1),  # one split walks 157 tiles of 157 pages: the table is read in batches of 32
])
def test_paged_cache_equals_contiguous_cache(ops, gpu_device, page, pages_per_seq, lengths, num_splits):
    """Scattered pages (shuffled block table, spare pages holding NaN) give the bits of the same rows
    in a contiguous cache, match the oracle, and only the appended rows change."""
    batch, capacity = len(lengths), page * pages_per_seq
    q, kcache, vcache, knew, vnew = make_case(300 + page, batch, capacity, fill=lengths)
    old = torch.tensor(lengths, dtype=torch.int32)
    generator = torch.Generator().manual_seed(page)
    pool = batch * pages_per_seq + 3
    table = torch.randperm(pool, generator=generator)[:batch * pages_per_seq].view(batch, pages_per_seq).to(torch.int32)
    paged_k = torch.full((pool, page, 8, 128), float("nan"), dtype=torch.bfloat16)
    paged_v = torch.full((pool, page, 8, 128), float("nan"), dtype=torch.bfloat16)
    paged_k[table.long()] = kcache.unflatten(1, (pages_per_seq, page))
    paged_v[table.long()] = vcache.unflatten(1, (pages_per_seq, page))
    want_o, want_lse, want_k, want_v = oracle.decode_step_indexed(q, paged_k, paged_v, knew, vnew, old, block_table=table)
    got_o, got_lse, got_k, got_v = run_indexed(ops, gpu_device, q, paged_k, paged_v, knew, vnew, old, capacity,
                                               num_splits, block_table=table)
    oracle.check_outputs(got_o, got_lse, want_o, want_lse)
    assert torch.equal(bits(got_k), bits(want_k)) and torch.equal(bits(got_v), bits(want_v))
    flat_o, flat_lse, _, _, _ = run_step(ops, gpu_device, q, kcache, vcache, knew, vnew, old, num_splits=num_splits)
    assert torch.equal(bits(got_o), bits(flat_o)) and torch.equal(got_lse.view(torch.int32), flat_lse.view(torch.int32))


def test_cache_batch_index(ops, gpu_device):
    batch, capacity, slots = 3, 512, 6
    q, kcache, vcache, knew, vnew = make_case(41, slots, capacity)
    q, knew, vnew = q[:batch], knew[:batch], vnew[:batch]
    index = torch.tensor([4, 0, 5], dtype=torch.int32)
    old = torch.tensor([511, 100, 0], dtype=torch.int32)
    want_o, want_lse, want_k, want_v = oracle.decode_step_indexed(q, kcache, vcache, knew, vnew, old, cache_batch_idx=index)
    got_o, got_lse, got_k, got_v = run_indexed(ops, gpu_device, q, kcache, vcache, knew, vnew, old, capacity,
                                               cache_batch_idx=index)
    oracle.check_outputs(got_o, got_lse, want_o, want_lse)
    assert torch.equal(bits(got_k), bits(want_k)) and torch.equal(bits(got_v), bits(want_v))
    flat_o, flat_lse, _, _, _ = run_step(ops, gpu_device, q, kcache[index.long()], vcache[index.long()], knew, vnew, old)
    assert torch.equal(bits(got_o), bits(flat_o)) and torch.equal(got_lse.view(torch.int32), flat_lse.view(torch.int32))


def test_indexed_argument_checks(ops, gpu_device):
    q, kcache, vcache, knew, vnew = (t.to(gpu_device) for t in make_case(1, 1, 128))
    old = torch.tensor([5], dtype=torch.int32, device=gpu_device)
    out, lse = torch.empty_like(q), torch.empty((1, 32, 1), device=gpu_device)
    ws = [torch.empty(n, device=gpu_device) for n in ops.indexed_workspace_spec(1, 128, 8, gpu_device.index)[1:3]]
    table = torch.zeros((1, 1), dtype=torch.int32, device=gpu_device)
    index = torch.zeros((1,), dtype=torch.int32, device=gpu_device)
    with pytest.raises(RuntimeError, match="exactly one"):
        ops.indexed_forward_out(q, kcache, vcache, knew, vnew, old, out, lse, *ws, 0, 1, True)
    with pytest.raises(RuntimeError, match="exactly one"):
        ops.indexed_forward_out(q, kcache, vcache, knew, vnew, old, out, lse, *ws, 0, 1, True, table, index)
    odd_k, odd_v = kcache[:, :96].contiguous(), vcache[:, :96].contiguous()
    with pytest.raises(RuntimeError, match="multiple of 64"):
        ops.indexed_forward_out(q, odd_k, odd_v, knew, vnew, old, out, lse, *ws, 0, 1, True, block_table=table)
    torch.cuda.synchronize()


@pytest.mark.parametrize("batch,capacity,lengths,num_splits", [
    (1, 256, [130], 0),
    (4, 1024, [1023, 0, 511, 64], 0),
    (2, 8192, [8191, 4000], 3),
])
def test_rotary_embedding_inside_the_launch(ops, gpu_device, batch, capacity, lengths, num_splits):
    """Un-rotated q / knew + RoPE tables give exactly what the plain entry point gives on inputs rotated
    (and re-rounded to BF16) on the host: same O and LSE bits, and the appended K row is the rotated row."""
    q, kcache, vcache, knew, vnew = make_case(500 + capacity, batch, capacity, fill=lengths)
    old = torch.tensor(lengths, dtype=torch.int32)
    cos, sin = oracle.rope_tables(capacity)
    want_o, want_lse, want_k, want_v = oracle.decode_step_rope(q, kcache, vcache, knew, vnew, old, cos, sin)
    device = gpu_device
    dq, dk, dv, dkn, dvn, dold = (t.to(device) for t in (q, kcache, vcache, knew, vnew, old))
    out = torch.full_like(dq, float("nan"))
    lse = torch.full((batch, 32, 1), float("nan"), device=device, dtype=torch.float32)
    spec = ops.workspace_spec(dq, dk, dold, num_splits, 1, True)
    ws = [torch.full((n,), float("nan"), device=device, dtype=torch.float32) for n in spec[1:3]]
    ops.rope_forward_out(dq, dk, dv, dkn, dvn, dold, out, lse, *ws, num_splits, 1, True, cos.to(device), sin.to(device))
    torch.cuda.synchronize()
    assert ops.library.device_status(device.index) == 0
    oracle.check_outputs(out.cpu(), lse.cpu(), want_o, want_lse)
    assert torch.equal(bits(dk.cpu()), bits(want_k)) and torch.equal(bits(dv.cpu()), bits(want_v))
    position = old.long()
    pc, ps = cos[position][:, None, None, :], sin[position][:, None, None, :]
    flat_o, flat_lse, _, _, _ = run_step(ops, device, oracle.rope_rotate(q, pc, ps), kcache, vcache,
                                         oracle.rope_rotate(knew, pc, ps), vnew, old, num_splits=num_splits)
    assert torch.equal(bits(out.cpu()), bits(flat_o)) and torch.equal(lse.cpu().view(torch.int32), flat_lse.view(torch.int32))


def test_in_launch_exchange_with_one_rank(ops, gpu_device):
    """The fused exchange route with a world of one: three consecutive steps (both slot parities and a
    reused slot) must equal the plain entry point bit for bit."""
    from tilecadence_b200 import sharding

    batch, capacity = 2, 1024
    q, kcache, vcache, knew, vnew = make_case(21, batch, capacity)
    device = gpu_device
    dq, dkn, dvn = q.to(device), knew.to(device), vnew.to(device)
    driver = sharding.ShardedDecode(ops, 0, 1, batch, capacity, device, exchange="peer")
    try:
        dk, dv = kcache.to(device), vcache.to(device)
        ref_k, ref_v = kcache.clone(), vcache.clone()
        for step, lengths in enumerate([[700, 3], [701, 4], [702, 5]]):
            old = torch.tensor(lengths, dtype=torch.int32)
            want_o, want_lse, ref_k, ref_v, _ = run_step(ops, device, q, ref_k, ref_v, knew, vnew, old)
            out = torch.full_like(dq, float("nan"))
            lse = torch.full((batch, 32, 1), float("nan"), device=device, dtype=torch.float32)
            driver.step(dq, dk, dv, dkn, dvn, old.to(device), out, lse)
            torch.cuda.synchronize()
            assert ops.library.device_status(device.index) == 0
            assert torch.equal(bits(out.cpu()), bits(want_o)), step
            assert torch.equal(lse.cpu().view(torch.int32), want_lse.view(torch.int32)), step
            assert torch.equal(bits(dk.cpu()), bits(ref_k)) and torch.equal(bits(dv.cpu()), bits(ref_v))
    finally:
        driver.close()


def test_missing_rank_ends_the_exchange_with_a_status(ops, gpu_device):
    """Failure detection without a fault: rank 0 of a world of two runs alone (rank 1's exchange block is a
    second block on this GPU that nobody fills). Its bounded wait expires, the kernel returns, the status
    word reports it, and the next ordinary call on the same context is correct."""
    import ctypes

    library, device = ops.library, gpu_device
    batch, capacity = 1, 256
    q, kcache, vcache, knew, vnew = make_case(31, batch, capacity)
    old = torch.tensor([100], dtype=torch.int32)
    size = ctypes.c_int64(0)
    library.call("tc_peer_block_bytes", batch, 8, 2, ctypes.byref(size))
    blocks = []
    try:
        for _ in range(2):
            block, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
            library.call("tc_peer_block_create", device.index, size.value, ctypes.byref(block), handle)
            blocks.append(block.value)
        table = (ctypes.c_void_p * 2)(*blocks)
        dq, dkn, dvn, dold = q.to(device), knew.to(device), vnew.to(device), old.to(device)
        dk, dv = kcache[:, :128].contiguous().to(device), vcache[:, :128].contiguous().to(device)
        out = torch.empty_like(dq)
        lse = torch.empty((batch, 32, 1), device=device, dtype=torch.float32)
        spec = ops.workspace_spec(dq, dk, dold, 0, 1, True)
        ws = [torch.empty(n, device=device, dtype=torch.float32) for n in spec[1:3]]
        # blocks smaller than this call's geometry needs are refused before anything is launched
        with pytest.raises(RuntimeError, match="too small"):
            ops.exchange_out(dq, dk, dv, dkn, dvn, dold, out, lse, *ws, 0, 1, True, 0, 0, table, size.value - 256)
        ops.exchange_out(dq, dk, dv, dkn, dvn, dold, out, lse, *ws, 0, 1, True, 0, 0, table, size.value)
        torch.cuda.synchronize()
        assert library.device_status(device.index) == 5   # "a rank never delivered"
        assert library.device_status(device.index) == 0   # reading clears it
    finally:
        torch.cuda.synchronize()
        for block in blocks:
            library.call("tc_peer_block_destroy", device.index, block)
    want_o, want_lse, _, _ = oracle.decode_step(q, kcache, vcache, knew, vnew, old)
    got_o, got_lse, _, _, _ = run_step(ops, device, q, kcache, vcache, knew, vnew, old)
    oracle.check_outputs(got_o, got_lse, want_o, want_lse)


@pytest.mark.parametrize("batch,capacity,base", [(1, 4096, 2045), (1, 16384, 12283), (2, 2048, 60)])
def test_consecutive_steps_on_one_cache_may_overlap_under_the_prefix_promise(ops, gpu_device, batch, capacity, base):
    """Twelve decode steps back to back on the same caches (each appends one row; the lengths of every step
    are a tensor of their own). Launched with the prefix promise, a step streams the rows below the row its
    predecessor appended while that predecessor is still finishing; outputs, LSE and the final caches must
    equal, bit for bit, those of the same chain launched without any promise. Lengths cross tile boundaries."""
    device, steps = gpu_device, 12
    _, kcache, vcache, _, _ = make_case(51, batch, capacity)
    q = oracle.seeded_normal(52, (steps, batch, 1, 32, 128))[0].to(device)
    knew, vnew = (t.to(device) for t in oracle.seeded_normal(53, (steps, batch, 1, 8, 128), (steps, batch, 1, 8, 128)))
    lengths = [torch.tensor([base + t - 17 * b for b in range(batch)], dtype=torch.int32, device=device)
               for t in range(steps)]
    results = {}
    for promise in (False, "prefix"):
        dk, dv = kcache.to(device), vcache.to(device)
        outs = torch.full((steps, batch, 1, 32, 128), float("nan"), device=device, dtype=torch.bfloat16)
        lses = torch.full((steps, batch, 32, 1), float("nan"), device=device)
        spec = ops.workspace_spec(q[0], dk, lengths[0], 0, 1, True)
        ws = [torch.empty(n, device=device, dtype=torch.float32) for n in spec[1:3]]
        torch.cuda.synchronize()
        for t in range(steps):
            ops.forward_out(q[t], dk, dv, knew[t], vnew[t], lengths[t], outs[t], lses[t], *ws, 0, 1, True,
                            cache_stable=promise)
        torch.cuda.synchronize()
        assert ops.library.device_status(device.index) == 0
        results[promise] = (outs.cpu(), lses.cpu(), dk.cpu(), dv.cpu())
    plain, early = results[False], results["prefix"]
    assert not torch.isnan(plain[0].float()).any()
    assert torch.equal(bits(plain[0]), bits(early[0])) and torch.equal(plain[1].view(torch.int32), early[1].view(torch.int32))
    assert torch.equal(bits(plain[2]), bits(early[2])) and torch.equal(bits(plain[3]), bits(early[3]))
    # and the last step agrees with the oracle on the caches as the chain left them before it
    host_k, host_v = kcache.clone(), vcache.clone()
    for t in range(steps - 1):
        for b in range(batch):
            host_k[b, int(lengths[t][b])] = knew[t, b, 0].cpu()
            host_v[b, int(lengths[t][b])] = vnew[t, b, 0].cpu()
    want_o, want_lse, want_k, want_v = oracle.decode_step(q[-1].cpu(), host_k, host_v, knew[-1].cpu(), vnew[-1].cpu(),
                                                          lengths[-1].cpu())
    oracle.check_outputs(early[0][-1], early[1][-1], want_o, want_lse)
    assert torch.equal(bits(early[2]), bits(want_k)) and torch.equal(bits(early[3]), bits(want_v))


def test_steps_on_different_caches_may_overlap_under_the_cache_stable_promise(ops, gpu_device):
    """Decode steps of eight different caches back to back (the layers of a model): with the cache-stable promise
    each step prefetches its whole share of its cache while the step before it runs. Same bits as without."""
    device, layers, capacity = gpu_device, 8, 8192
    old = torch.tensor([capacity - 100], dtype=torch.int32, device=device)
    prefix = [oracle.seeded_normal(60 + layer, (1, capacity, 8, 128), (1, capacity, 8, 128)) for layer in range(layers)]
    q, knew, vnew = (t.to(device) for t in oracle.seeded_normal(61, (1, 1, 32, 128), (1, 1, 8, 128), (1, 1, 8, 128)))
    results = {}
    for promise in (False, True):
        caches = [(k.to(device), v.to(device)) for k, v in prefix]
        outs = torch.full((layers, 1, 1, 32, 128), float("nan"), device=device, dtype=torch.bfloat16)
        lses = torch.full((layers, 1, 32, 1), float("nan"), device=device)
        spec = ops.workspace_spec(q, caches[0][0], old, 0, 1, True)
        ws = [torch.empty(n, device=device, dtype=torch.float32) for n in spec[1:3]]
        torch.cuda.synchronize()
        for repeat in range(3):
            for layer in range(layers):
                ops.forward_out(q, *caches[layer], knew, vnew, old, outs[layer], lses[layer], *ws, 0, 1, True,
                                cache_stable=promise)
        torch.cuda.synchronize()
        assert ops.library.device_status(device.index) == 0
        results[promise] = (outs.cpu(), lses.cpu(), [k[:, capacity - 100].cpu() for k, _ in caches])
    plain, early = results[False], results[True]
    assert torch.equal(bits(plain[0]), bits(early[0])) and torch.equal(plain[1].view(torch.int32), early[1].view(torch.int32))
    for a, b in zip(plain[2], early[2]):
        assert torch.equal(bits(a), bits(b))
    want_o, want_lse, _, _ = oracle.decode_step(q.cpu(), prefix[3][0], prefix[3][1], knew.cpu(), vnew.cpu(), old.cpu())
    oracle.check_outputs(early[0][3], early[1][3], want_o, want_lse)


def test_argument_checks(ops, gpu_device):
    q, kcache, vcache, knew, vnew = (t.to(gpu_device) for t in make_case(1, 1, 128))
    old = torch.zeros(1, dtype=torch.int32, device=gpu_device)
    out, lse = torch.empty_like(q), torch.empty((1, 32, 1), device=gpu_device)
    spec = ops.workspace_spec(q, kcache, old, 0, 1, True)
    ws = [torch.empty(n, device=gpu_device) for n in spec[1:]]
    with pytest.raises(RuntimeError, match="workspace is too small"):
        ops.forward_out(q, kcache, vcache, knew, vnew, old, out, lse, ws[0][:1], ws[1], 0, 1, True)
    with pytest.raises(RuntimeError, match="disjoint"):
        ops.forward_out(q, kcache, kcache, knew, vnew, old, out, lse, *ws, 0, 1, True)
    with pytest.raises(RuntimeError, match="old_lengths"):
        ops.forward_out(q, kcache, vcache, knew, vnew, old.long(), out, lse, *ws, 0, 1, True)
    with pytest.raises(RuntimeError, match="mapping"):
        ops.workspace_spec(q, kcache, old, 0, 2, True)
    with pytest.raises(RuntimeError, match="Contiguous BF16"):
        ops.workspace_spec(q.float(), kcache, old, 0, 1, True)
    resources = ops.resources(q, kcache, old, 0, 1, True)
    assert len(resources) == 34 and resources[12] == 160 and resources[19] >= 1 and resources[0] == spec[0]


def test_bound_call_repeats_the_validated_call(ops, gpu_device):
    q, kcache, vcache, knew, vnew = make_case(12, 1, 512)
    old = torch.tensor([300], dtype=torch.int32)
    want_o, want_lse, want_k, want_v = oracle.decode_step(q, kcache, vcache, knew, vnew, old)
    dq, dk, dv, dkn, dvn, dold = (t.to(gpu_device) for t in (q, kcache, vcache, knew, vnew, old))
    out, lse = torch.empty_like(dq), torch.empty((1, 32, 1), device=gpu_device)
    spec = ops.workspace_spec(dq, dk, dold, 0, 1, True)
    ws = [torch.empty(n, device=gpu_device) for n in spec[1:]]
    invoke = ops.bind_forward_out(dq, dk, dv, dkn, dvn, dold, out, lse, *ws, 0, 1, True)
    for _ in range(3):  # the append rewrites the same row with the same bits: repeatable
        invoke()
    torch.cuda.synchronize()
    oracle.check_outputs(out.cpu(), lse.cpu(), want_o, want_lse)
    assert torch.equal(bits(dk.cpu()), bits(want_k)) and torch.equal(bits(dv.cpu()), bits(want_v))
    with pytest.raises(RuntimeError, match="Invalid complete output"):
        ops.bind_forward_out(dq, dk, dv, dkn, dvn, dold, out.float(), lse, *ws, 0, 1, True)

"""The fused QKV projection + RMS norm + RoPE step (``tc_qkv_rope_forward_out``) against its CPU oracle.

The accumulation order of a 2560-term dot product differs between the tensor-core kernel and the host, so
the fp32 sums agree to rounding noise only and results are compared after the BF16 roundings with a
two-ulp bound (2^-7 relative to max(1, |expected|)); without norm and RoPE almost every element must be
bit-identical. The step's outputs then feed the decode operator, which must agree with the operator fed
by the oracle's outputs within the decode tolerances.
"""
import pytest
import torch

from oracle import attention as oracle
from tilecadence_b200 import cuda_runtime

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def project(library):
    return cuda_runtime.ops_for(library, "project")


def make_inputs(seed, tokens, hidden, q_heads=32, kv_heads=8):
    rows = (q_heads + 2 * kv_heads) * 128
    x, w, qn, kn = oracle.seeded_normal(seed, (tokens, hidden), (rows, hidden), (128,), (128,), dtype=torch.float32)
    w = (w / hidden ** 0.5).to(torch.bfloat16)
    return x.to(torch.bfloat16), w, (1 + 0.1 * qn).to(torch.bfloat16), (1 + 0.1 * kn).to(torch.bfloat16)


def run(project, device, x, w, positions, qn=None, kn=None, cos=None, sin=None):
    tokens = x.size(0)
    move = lambda t: None if t is None else t.to(device)
    outs = [torch.full((tokens, 1, heads, 128), float("nan"), device=device, dtype=torch.bfloat16)
            for heads in (project.q_heads, project.kv_heads, project.kv_heads)]
    project.forward_out(move(x), move(w), move(positions), *outs, q_norm_weight=move(qn), k_norm_weight=move(kn),
                        rope_cos=move(cos), rope_sin=move(sin))
    torch.cuda.synchronize()
    assert project.library.device_status(device.index) == 0
    return [t.cpu() for t in outs]


def close(got, want, exact_share):
    got, want = got.float(), want.float()
    assert torch.isfinite(got).all()
    assert ((got - want).abs() <= 2 ** -7 * want.abs().clamp_min(1.0)).all()
    assert (got == want).float().mean().item() >= exact_share


@pytest.mark.parametrize("tokens,hidden", [(1, 2560), (4, 2560), (8, 4096), (3, 64), (5, 192)])
def test_plain_projection(project, gpu_device, tokens, hidden):
    x, w, _, _ = make_inputs(10 + tokens, tokens, hidden)
    want = oracle.project_qkv_rope(x, w, None, 32, 8)
    got = run(project, gpu_device, x, w, None)
    for g, t in zip(got, want):
        close(g, t, 0.97)


@pytest.mark.parametrize("tokens", [1, 4])
def test_norm_and_rope_like_qwen3(project, gpu_device, tokens):
    x, w, qn, kn = make_inputs(20 + tokens, tokens, 2560)
    cos, sin = oracle.rope_tables(4096)
    positions = torch.tensor([4095, 0, 17, 1234][:tokens], dtype=torch.int32)
    want = oracle.project_qkv_rope(x, w, positions, 32, 8, qn, kn, cos, sin)
    got = run(project, gpu_device, x, w, positions, qn, kn, cos, sin)
    for g, t in zip(got, want):
        close(g, t, 0.85)


def test_feeds_the_decode_operator(project, library, gpu_device):
    """The projected q / knew / vnew go straight into the decode operator (same layout, no copy or cast):
    its result matches the oracle's decode of the same tensors, and the row appended to the K cache is the
    projected, normed and rotated K row."""
    tokens, capacity = 4, 512
    x, w, qn, kn = make_inputs(31, tokens, 2560)
    cos, sin = oracle.rope_tables(capacity)
    old = torch.tensor([100, 0, 511, 257], dtype=torch.int32)
    kcache, vcache = oracle.seeded_normal(32, (tokens, capacity, 8, 128), (tokens, capacity, 8, 128))
    q, knew, vnew = run(project, gpu_device, x, w, old, qn, kn, cos, sin)
    want_q, want_k, want_v = oracle.project_qkv_rope(x, w, old, 32, 8, qn, kn, cos, sin)
    for got, want in ((q, want_q), (knew, want_k), (vnew, want_v)):
        close(got, want, 0.85)
    want_o, want_lse, _, _ = oracle.decode_step(q, kcache, vcache, knew, vnew, old)
    decode = cuda_runtime.ops_for(library, "decode")
    device = gpu_device
    dq, dk, dv, dkn, dvn, dold = (t.to(device) for t in (q, kcache, vcache, knew, vnew, old))
    out, lse = torch.empty_like(dq), torch.empty((tokens, 32, 1), device=device, dtype=torch.float32)
    spec = decode.workspace_spec(dq, dk, dold, 0, 1, True)
    ws = [torch.empty(n, device=device, dtype=torch.float32) for n in spec[1:3]]
    decode.forward_out(dq, dk, dv, dkn, dvn, dold, out, lse, *ws, 0, 1, True)
    torch.cuda.synchronize()
    oracle.check_outputs(out.cpu(), lse.cpu(), want_o, want_lse)
    for b in range(tokens):
        assert torch.equal(dk[b, old[b]].cpu().view(torch.int16), knew[b, 0].view(torch.int16))


def test_decode_may_stream_the_cache_while_the_projection_finishes(project, library, gpu_device):
    """Projection -> decode chains on one stream, twenty layers' worth of them back to back with a
    different token slab each time: the decode step launched with the cache-stable promise (its K/V stream
    starts while the projection is still running) gives bit for bit the results, and the appended rows, of
    the plain step."""
    tokens, capacity, layers = 1, 8192, 20
    device = gpu_device
    decode = cuda_runtime.ops_for(library, "decode")
    cos, sin = (t.to(device) for t in oracle.rope_tables(capacity))
    old = torch.tensor([capacity - 2], dtype=torch.int32, device=device)
    slabs, weights = [], []
    for layer in range(layers):
        x, w, _, _ = make_inputs(200 + layer, tokens, 2560)
        slabs.append(x.to(device))
        weights.append(w.to(device))
    prefix_k, prefix_v = oracle.seeded_normal(77, (tokens, capacity, 8, 128), (tokens, capacity, 8, 128))
    results = {}
    for promise, early in ((False, False), (True, False), (True, True)):
        caches = [(prefix_k.to(device), prefix_v.to(device)) for _ in range(layers)]
        q, knew, vnew = (torch.empty((tokens, 1, h, 128), device=device, dtype=torch.bfloat16) for h in (32, 8, 8))
        outs = torch.full((layers, tokens, 1, 32, 128), float("nan"), device=device, dtype=torch.bfloat16)
        lses = torch.full((layers, tokens, 32, 1), float("nan"), device=device)
        spec = decode.workspace_spec(q, caches[0][0], old, 0, 1, True)
        ws = [torch.empty(n, device=device, dtype=torch.float32) for n in spec[1:3]]
        torch.cuda.synchronize()
        for layer in range(layers):
            project.forward_out(slabs[layer], weights[layer], old, q, knew, vnew, rope_cos=cos, rope_sin=sin,
                                release_early=early)
            decode.forward_out(q, *caches[layer], knew, vnew, old, outs[layer], lses[layer], *ws, 0, 1, True,
                               cache_stable=promise)
        torch.cuda.synchronize()
        assert library.device_status(device.index) == 0
        results[promise, early] = (outs.cpu(), lses.cpu(), [k[:, capacity - 2].cpu() for k, _ in caches])
    plain = results[False, False]
    assert not torch.isnan(plain[0].float()).any()
    # (every layer has a cache of its own here, so with the projection's early release the decode step of a layer
    # also streams beside the decode step of the layer before it without breaking its promise)
    for overlapped in (results[True, False], results[True, True]):
        assert torch.equal(plain[0].view(torch.int16), overlapped[0].view(torch.int16))
        assert torch.equal(plain[1].view(torch.int32), overlapped[1].view(torch.int32))
        for a, b in zip(plain[2], overlapped[2]):
            assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_a_chain_of_projections_released_early_gives_the_same_bits(project, library, gpu_device):
    """Thirty projections back to back on one stream, each with its own weights and token slab and its own
    outputs: with TC_PROJECT_RELEASE_EARLY a launch's weight stream starts while the launch two places before
    it is still running; every output must equal the plain chain's bit for bit."""
    tokens, layers = 4, 30
    device = gpu_device
    cos, sin = (t.to(device) for t in oracle.rope_tables(4096))
    positions = torch.tensor([5, 77, 1024, 4095], dtype=torch.int32, device=device)
    slabs, weights = [], []
    for layer in range(layers):
        x, w, _, _ = make_inputs(500 + layer, tokens, 2560)
        slabs.append(x.to(device))
        weights.append(w.to(device))
    ones = torch.ones(128, device=device, dtype=torch.bfloat16)
    results = {}
    for early in (False, True):
        outs = [[torch.full((tokens, 1, h, 128), float("nan"), device=device, dtype=torch.bfloat16) for h in (32, 8, 8)]
                for _ in range(layers)]
        torch.cuda.synchronize()
        for layer in range(layers):
            project.forward_out(slabs[layer], weights[layer], positions, *outs[layer], q_norm_weight=ones,
                                k_norm_weight=ones, rope_cos=cos, rope_sin=sin, release_early=early)
        torch.cuda.synchronize()
        assert library.device_status(device.index) == 0
        results[early] = [[t.cpu() for t in triple] for triple in outs]
    for plain, released in zip(results[False], results[True]):
        for a, b in zip(plain, released):
            assert not torch.isnan(a.float()).any()
            assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_argument_checks(project, gpu_device):
    x, w, _, _ = make_inputs(1, 2, 128)
    outs = [torch.empty((2, 1, h, 128), device=gpu_device, dtype=torch.bfloat16) for h in (32, 8, 8)]
    cos, sin = oracle.rope_tables(8)
    with pytest.raises(RuntimeError, match="tokens<=8"):
        project.forward_out(torch.zeros((9, 128), device=gpu_device, dtype=torch.bfloat16), w.to(gpu_device), None, *outs)
    with pytest.raises(RuntimeError, match="both RoPE"):
        project.forward_out(x.to(gpu_device), w.to(gpu_device), None, *outs, rope_cos=cos.to(gpu_device))
    with pytest.raises(RuntimeError, match="multiple of 64"):
        bad = torch.zeros((2, 96), device=gpu_device, dtype=torch.bfloat16)
        project.forward_out(bad, torch.zeros((6144, 96), device=gpu_device, dtype=torch.bfloat16), None, *outs)

"""The allocation-free decode entry point against the regular one, through the C ABI.

``tc_decode_forward_out_static`` serves callers that may not allocate device memory (a server whose
allocator owns every byte of a fixed budget, code that must not touch a caching allocator, call sites
that cannot afford cudaMalloc's synchronisation): it takes no workspace and keeps its split partials
in an array inside the library image. Both entry points run the same kernel with the same split count,
so their results are compared with the tolerances of the decode parity tests (O max-abs 2e-2, LSE
1e-3 relative, caches bit-exact). Two consecutive steps are run because the built-in array keeps the
first call's contents when the second call starts.

Collected last so that a run stopping at the first failure has already run every other test.
"""
import ctypes

import pytest
import torch

from oracle import attention as oracle
from tilecadence_b200 import cuda_runtime

pytestmark = pytest.mark.gpu


def pointer(tensor):
    return ctypes.c_void_p(tensor.data_ptr())


def stream_of(tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(tensor.device).cuda_stream)


def call_static(library, q, kcache, vcache, knew, vnew, old, out, lse, num_splits=0, mapping=1, append=True):
    library.call("tc_decode_forward_out_static", q.device.index, stream_of(q), pointer(q), pointer(kcache),
                 pointer(vcache), pointer(knew), pointer(vnew), pointer(old), pointer(out), pointer(lse),
                 q.size(0), kcache.size(1), kcache.size(2), num_splits, mapping, int(append))


def call_regular(library, q, kcache, vcache, knew, vnew, old, out, lse, num_splits=0, mapping=1, append=True):
    spec = (ctypes.c_int64 * 3)()
    library.call("tc_decode_workspace_spec", q.device.index, q.size(0), kcache.size(1), kcache.size(2), num_splits,
                 mapping, int(append), spec)
    ws_o = torch.empty(spec[1], device=q.device, dtype=torch.float32)
    ws_lse = torch.empty(spec[2], device=q.device, dtype=torch.float32)
    library.call("tc_decode_forward_out", q.device.index, stream_of(q), pointer(q), pointer(kcache), pointer(vcache),
                 pointer(knew), pointer(vnew), pointer(old), pointer(out), pointer(lse), pointer(ws_o), ws_o.numel(),
                 pointer(ws_lse), ws_lse.numel(), q.size(0), kcache.size(1), kcache.size(2), num_splits, mapping,
                 int(append))


@pytest.mark.parametrize("batch,capacity,start", [(1, 4096, 3000), (4, 1024, 500)])
def test_static_entry_matches_regular_entry_on_two_steps(library, gpu_device, batch, capacity, start):
    device = gpu_device
    prefix_k, prefix_v = oracle.seeded_normal(77 + batch, (batch, capacity, 8, 128), (batch, capacity, 8, 128))
    steps = [oracle.seeded_normal(90 + s, (batch, 1, 32, 128), (batch, 1, 8, 128), (batch, 1, 8, 128)) for s in range(2)]
    caches = {name: (prefix_k.to(device), prefix_v.to(device)) for name in ("static", "regular")}
    host_k, host_v = prefix_k, prefix_v
    for step, (q, knew, vnew) in enumerate(steps):
        dq, dkn, dvn = q.to(device), knew.to(device), vnew.to(device)
        lengths = torch.tensor([start + step - 7 * b for b in range(batch)], dtype=torch.int32)
        old = lengths.to(device)
        results = {}
        for name, call in (("static", call_static), ("regular", call_regular)):
            out = torch.full_like(dq, float("nan"))
            lse = torch.full((batch, 32, 1), float("nan"), device=device, dtype=torch.float32)
            call(library, dq, *caches[name], dkn, dvn, old, out, lse)
            torch.cuda.synchronize()
            results[name] = (out.cpu(), lse.cpu())
        oracle.check_outputs(results["static"][0], results["static"][1], results["regular"][0].float(),
                             results["regular"][1])
        for a, b in zip(caches["static"], caches["regular"]):
            assert torch.equal(a.view(torch.int16), b.view(torch.int16))
        # and both agree with the CPU oracle, whose caches advance with the same appends
        want_o, want_lse, host_k, host_v = oracle.decode_step(q, host_k, host_v, knew, vnew, lengths)
        oracle.check_outputs(results["static"][0], results["static"][1], want_o, want_lse)
        assert torch.equal(caches["static"][0].cpu().view(torch.int16), host_k.view(torch.int16))
        assert torch.equal(caches["static"][1].cpu().view(torch.int16), host_v.view(torch.int16))
    assert library.device_status(device.index) == 0


def test_static_entry_rejects_sizes_beyond_its_scratch(library, gpu_device):
    device = gpu_device
    batch = 5  # 5 * 32 = 160 rows > 128
    q = torch.zeros((batch, 1, 32, 128), device=device, dtype=torch.bfloat16)
    cache_k = torch.zeros((batch, 128, 8, 128), device=device, dtype=torch.bfloat16)
    cache_v = torch.zeros_like(cache_k)
    new_k = torch.zeros((batch, 1, 8, 128), device=device, dtype=torch.bfloat16)
    new_v = torch.zeros_like(new_k)
    old = torch.zeros(batch, device=device, dtype=torch.int32)
    out, lse = torch.empty_like(q), torch.empty((batch, 32, 1), device=device)
    with pytest.raises(RuntimeError, match="exceeds the built-in scratch"):
        call_static(library, q, cache_k, cache_v, new_k, new_v, old, out, lse)
    with pytest.raises(RuntimeError, match="splits exceed the built-in scratch"):
        call_static(library, q[:1], cache_k[:1], cache_v[:1], new_k[:1], new_v[:1], old[:1], out[:1], lse[:1],
                    num_splits=64)

"""The allocation-free decode entry point against the regular one, through the C ABI.

``tc_decode_forward_out_static`` serves callers that may not allocate device memory (a server whose
allocator owns every byte of a fixed budget, code that must not touch a caching allocator, call sites
that cannot afford cudaMalloc's synchronisation): it takes no workspace and keeps its split partials
in an array inside the library image. Both entry points run the same kernel with the same split count,
so their results are compared with the tolerances of the decode parity tests (O max-abs 2e-2, LSE
1e-3 relative, caches bit-exact). Two consecutive steps are run because the built-in array keeps the
first call's contents when the second call starts.

The status word of a static call sits in that same array; ``tc_device_status`` and
``tc_decode_static_status_word`` are the two documented ways to reach it, and neither allocates.

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


def static_status_word(library, device):
    word = ctypes.c_void_p()
    library.call("tc_decode_static_status_word", device.index, ctypes.byref(word))
    assert word.value
    return word


def test_static_status_word_is_what_device_status_reads(library, gpu_device):
    """A code left in the static array's status word (here put there by the test with a 4-byte copy, standing
    in for a kernel whose bounded wait ran out) comes back from tc_device_status exactly once."""
    device = gpu_device
    cudart = ctypes.CDLL("libcudart.so.12")
    cudart.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
    with torch.cuda.device(device):
        word = static_status_word(library, device)
        assert library.device_status(device.index) == 0
        code = ctypes.c_int32(2)  # what the kernel stores when a consumer's wait for a K/V stage expires
        assert cudart.cudaMemcpy(word, ctypes.byref(code), 4, 1) == 0  # host -> device
        assert library.device_status(device.index) == 2
        assert library.device_status(device.index) == 0  # reading cleared it
        seen = ctypes.c_int32(-1)
        assert cudart.cudaMemcpy(ctypes.byref(seen), word, 4, 2) == 0  # device -> host
        assert seen.value == 0


def test_static_entry_and_its_status_readers_allocate_nothing(library, gpu_device):
    """Free device memory is the same before and after a warmed-up static call and both status readers."""
    device = gpu_device
    batch, capacity = 2, 2048
    prefix_k, prefix_v = oracle.seeded_normal(5, (batch, capacity, 8, 128), (batch, capacity, 8, 128))
    q, knew, vnew = oracle.seeded_normal(6, (batch, 1, 32, 128), (batch, 1, 8, 128), (batch, 1, 8, 128))
    dk, dv, dq, dkn, dvn = (t.to(device) for t in (prefix_k, prefix_v, q, knew, vnew))
    old = torch.tensor([1500, 900], dtype=torch.int32, device=device)
    old_next = old + 1  # made before the measurement: creating a tensor may make torch's allocator grow
    out = torch.empty_like(dq)
    lse = torch.empty((batch, 32, 1), device=device, dtype=torch.float32)
    call_static(library, dq, dk, dv, dkn, dvn, old, out, lse)  # first call: address look-up, kernel load
    static_status_word(library, device)
    library.device_status(device.index)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(device)
    call_static(library, dq, dk, dv, dkn, dvn, old_next, out, lse)
    static_status_word(library, device)
    assert library.device_status(device.index) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(device)
    assert free_after == free_before


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
    misaligned = torch.empty(33, device=device, dtype=torch.float32).view(torch.uint8)[1:129].view(torch.uint8)
    with pytest.raises(RuntimeError, match="misaligned old_lengths or LSE"):
        library.call("tc_decode_forward_out_static", device.index, stream_of(q), pointer(q[:1]), pointer(cache_k[:1]),
                     pointer(cache_v[:1]), pointer(new_k[:1]), pointer(new_v[:1]), pointer(old[:1]), pointer(out[:1]),
                     ctypes.c_void_p(misaligned.data_ptr()), 1, 128, 8, 0, 1, 1)

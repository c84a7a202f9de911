"""The generated two-tile kernels against the CPU oracle, through the emitter, nvcc and the C ABI.

Config 1 of the benchmark set: batch 1, 8 heads, 64 tokens, D128, FP16, non-causal, N(0,1) from seed 0
(the golden case of ``tests/golden/attention_golden.npz``); plus BF16 and causal variants. Tolerances:
O max-abs <= 1e-2 (FP16) / 2e-2 (BF16), LSE <= 1e-3 relative; every exchange arm must equal the
``retain`` arm bit for bit (``tilecadence/bench_exchange.py:96-113``).
"""
import pytest
import torch

from oracle import attention as oracle
from tilecadence_b200 import cuda_runtime, exchange, model
from tilecadence_b200.emit_exchange import RESOURCE_KEYS, emit

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def arm_ops(tmp_path_factory):
    built = {}
    for arm in exchange.ARMS:
        problem = exchange.build_problem(arm)
        result = model.solve(problem, max_time_seconds=2)
        directory = tmp_path_factory.mktemp(arm) / "emitted"
        emit(problem, result, directory)
        built[arm], receipt = cuda_runtime.build_cuda(directory, None, "cuda:0")
        assert built[arm].phase == "exchange" and receipt["target"] == "sm_100a"
    return built


def run(ops, device, q, k, v, causal):
    dq, dk, dv = q.to(device), k.to(device), v.to(device)
    out = torch.full_like(dq, float("nan"))
    lse = torch.full((q.size(0), q.size(2), 64), float("nan"), device=device, dtype=torch.float32)
    ops.forward_out(dq, dk, dv, out, lse, None, causal, True, False)
    torch.cuda.synchronize()
    assert ops.library.device_status(device.index) == 0
    return out.cpu(), lse.cpu()


@pytest.mark.parametrize("dtype,causal,batch,heads,seed", [
    (torch.float16, False, 1, 8, 0),   # config 1
    (torch.float16, True, 1, 8, 0),
    (torch.bfloat16, False, 2, 5, 3),
    (torch.bfloat16, True, 2, 5, 3),
])
def test_arms_match_oracle_and_each_other(arm_ops, gpu_device, dtype, causal, batch, heads, seed):
    q, k, v = oracle.seeded_normal(seed, (batch, 64, heads, 128), (batch, 64, heads, 128), (batch, 64, heads, 128),
                                   dtype=dtype)
    want_o, want_lse = oracle.attention(q, k, v, causal=causal)
    results = {arm: run(ops, gpu_device, q, k, v, causal) for arm, ops in arm_ops.items()}
    oracle.check_outputs(*results["retain"], want_o, want_lse, dtype=dtype)
    for arm in ("one", "multi", "relocated_two_p"):
        assert torch.equal(results[arm][0].view(torch.int16), results["retain"][0].view(torch.int16)), arm
        assert torch.equal(results[arm][1].view(torch.int32), results["retain"][1].view(torch.int32)), arm


def test_default_library_carries_the_committed_plan(library, gpu_device):
    ops = cuda_runtime.ops_for(library, "exchange")
    q, k, v = oracle.seeded_normal(0, (1, 64, 8, 128), (1, 64, 8, 128), (1, 64, 8, 128), dtype=torch.float16)
    got = run(ops, gpu_device, q, k, v, False)
    oracle.check_outputs(*got, *oracle.attention(q, k, v, causal=False), dtype=torch.float16)
    resources = dict(zip(RESOURCE_KEYS, ops.resources(q.to(gpu_device), False), strict=True))
    assert resources["threads"] == 128 and resources["dynamic_shared_bytes"] == 32768 + 1024
    assert resources["theoretical_active_ctas_per_sm"] >= 1 and resources["required_nonce_elements"] == 0
    out, lse = ops.forward(q.to(gpu_device), k.to(gpu_device), v.to(gpu_device), None, False)
    torch.cuda.synchronize()
    assert torch.equal(out.cpu().view(torch.int16), got[0].view(torch.int16))
    with pytest.raises(RuntimeError, match=r"\[B,64,H,128\]"):
        ops.forward(q[:, :32].to(gpu_device), k[:, :32].to(gpu_device), v[:, :32].to(gpu_device), None, False)

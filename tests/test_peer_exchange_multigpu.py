"""Fused cross-GPU decode exchange on two or more GPUs of one node (skipped with fewer).

One process per GPU. Every rank keeps a KV-sequence shard, runs ``tc_decode_exchange_out`` (partials
cross NVLink as plain peer stores inside the decode launch) and must end with the full result:
within tolerance of the CPU oracle, and bit-identical to merging the same shards' partials with the
standalone combine kernel on one GPU. Several consecutive steps exercise both slot parities.
"""
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank, world, port, results):
    import torch.distributed as dist

    from oracle import attention as oracle
    from tilecadence_b200 import cuda_runtime, sharding

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    driver = None
    try:
        device = torch.device("cuda", rank)
        torch.cuda.set_device(device)
        ops = cuda_runtime.ops_for(cuda_runtime.default_library(), "decode")
        batch, capacity = 4, 256 * world
        kcache, vcache, q, knew, vnew = oracle.seeded_normal(
            77, (batch, capacity, 8, 128), (batch, capacity, 8, 128), (batch, 1, 32, 128), (batch, 1, 8, 128),
            (batch, 1, 8, 128))
        start, length = sharding.kv_sequence_shard(rank, world, capacity)
        dq, dkn, dvn = q.to(device), knew.to(device), vnew.to(device)
        shards = [(kcache[:, s * length:(s + 1) * length].contiguous().to(device),
                   vcache[:, s * length:(s + 1) * length].contiguous().to(device)) for s in range(world)]
        mine = tuple(t.clone() for t in shards[rank])
        driver = sharding.ShardedDecode(ops, rank, world, batch, capacity, device, exchange="peer")
        ref_k, ref_v = kcache.clone(), vcache.clone()
        lengths = torch.tensor([capacity - 4, 3, length - 1, length + 7], dtype=torch.int32)
        for step in range(4):
            old = lengths + step
            want_o, want_lse, ref_k, ref_v = oracle.decode_step(q, ref_k, ref_v, knew, vnew, old)
            dold = old.to(device)
            out = torch.full_like(dq, float("nan"))
            lse = torch.full((batch, 32, 1), float("nan"), device=device, dtype=torch.float32)
            driver.step(dq, mine[0], mine[1], dkn, dvn, dold, out, lse)
            # the same step from all shards on this GPU alone, merged by the standalone kernel
            part_o = torch.empty((world, batch * 32, 128), device=device, dtype=torch.float32)
            part_lse = torch.empty((world, batch * 32), device=device, dtype=torch.float32)
            for s, (dk, dv) in enumerate(shards):
                spec = ops.workspace_spec(dq, dk, dold, 0, 1, True)
                ws = [torch.empty(n, device=device, dtype=torch.float32) for n in spec[1:3]]
                ops.partial_out(dq, dk, dv, dkn, dvn, dold, part_o[s], part_lse[s], *ws, 0, 1, True, s * length)
            local_o, local_lse = torch.empty_like(out), torch.empty_like(lse)
            ops.combine_partials(part_o, part_lse, local_o, local_lse)
            torch.cuda.synchronize(device)
            assert ops.library.device_status(device.index) == 0
            oracle.check_outputs(out.cpu(), lse.cpu(), want_o, want_lse)
            assert torch.equal(out.view(torch.int16), local_o.view(torch.int16)), step
            assert torch.equal(lse.view(torch.int32), local_lse.view(torch.int32)), step
            for got, want in ((mine[0], ref_k), (mine[1], ref_v)):
                assert torch.equal(got.cpu().view(torch.int16), want[:, start:start + length].view(torch.int16))
        results[rank] = "ok"
    finally:
        if driver is not None:
            driver.close()
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_exchange_across_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(worker, args=(world, free_port(), results), nprocs=world, join=True)
    assert dict(results) == {rank: "ok" for rank in range(world)}

"""Host logic of the multi-GPU drivers on CPU ranks (gloo, world size 2).

The CUDA operators are replaced by a stand-in that computes the same partials with the CPU
oracle, so what is under test is the orchestration: shard ownership, which rank appends, the packed
all-gather layout and the merge order. The product path never uses such a stand-in.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import attention as oracle
from tilecadence_b200 import sharding


class OracleOps:
    """Stand-in with the decode operator's interface, backed by the CPU oracle (tests only)."""

    def workspace_spec(self, q, kcache, old_lengths, num_splits, mapping, append):
        return [1, 0, 0]

    def partial_out(self, q, kcache, vcache, knew, vnew, old_lengths, partial_o, partial_lse, ws_o, ws_lse,
                    num_splits, mapping, append, kv_shard_start):
        out, lse, kafter, vafter = oracle.decode_step(q, kcache, vcache, knew, vnew, old_lengths, append=append,
                                                      shard_start=kv_shard_start, partial=True)
        kcache.copy_(kafter)
        vcache.copy_(vafter)
        partial_o.copy_(out.reshape(partial_o.shape))
        partial_lse.copy_(lse.reshape(partial_lse.shape))

    def combine_partials(self, partial_o, partial_lse, out, lse):
        merged, merged_lse = oracle.combine(partial_o, partial_lse)
        out.copy_(merged.reshape(out.shape).to(out.dtype))
        lse.copy_(merged_lse.reshape(lse.shape))


def free_port():
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        batch, capacity = 2, 96
        kcache, vcache, q, knew, vnew = oracle.seeded_normal(21, (batch, capacity, 8, 128), (batch, capacity, 8, 128),
                                                             (batch, 1, 32, 128), (batch, 1, 8, 128), (batch, 1, 8, 128))
        old = torch.tensor([70, 3], dtype=torch.int32)
        want_o, want_lse, want_k, want_v = oracle.decode_step(q, kcache, vcache, knew, vnew, old)
        start, length = sharding.kv_sequence_shard(rank, world, capacity)
        kshard, vshard = kcache[:, start:start + length].clone(), vcache[:, start:start + length].clone()
        driver = sharding.ShardedDecode(OracleOps(), rank, world, batch, capacity, torch.device("cpu"))
        out = torch.empty((batch, 1, 32, 128), dtype=torch.bfloat16)
        lse = torch.empty((batch, 32, 1), dtype=torch.float32)
        driver.step(q, kshard, vshard, knew, vnew, old, out, lse)
        oracle.check_outputs(out, lse, want_o, want_lse)
        assert torch.equal(kshard.view(torch.int16), want_k[:, start:start + length].view(torch.int16))
        assert torch.equal(vshard.view(torch.int16), want_v[:, start:start + length].view(torch.int16))
        # rank 1 owns row 70 of sequence 0, rank 0 owns row 3 of sequence 1: each appended exactly one row
        changed = (kshard.view(torch.int16) != kcache[:, start:start + length].view(torch.int16)).any(dim=(2, 3))
        assert changed.sum().item() == 1 and changed[1 - rank, (70 if rank else 3) - start]
        # sequence 1 has no visible key on rank 1: its partial LSE is -inf
        _, gathered_lse = driver.views(driver.gathered)
        assert torch.isinf(gathered_lse[1].view(batch, 32)[1]).all()
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_sharded_decode_two_ranks():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(worker, args=(world, free_port(), results), nprocs=world, join=True)
    assert dict(results) == {0: "ok", 1: "ok"}


def test_shard_arithmetic():
    assert sharding.kv_head_slice(1, 4) == (slice(2, 4), slice(8, 16))
    assert sharding.kv_head_slice(0, 1) == (slice(0, 8), slice(0, 32))
    assert sharding.kv_sequence_shard(3, 8, 32768) == (12288, 4096)
    with pytest.raises(ValueError):
        sharding.kv_head_slice(0, 3)
    with pytest.raises(ValueError):
        sharding.kv_sequence_shard(0, 3, 32768)


class FakePeerLibrary:
    """Stands in for the C-ABI library's exchange-block calls (no GPU): hands out fake addresses, and on
    the rank named ``fail_on`` refuses to map other ranks' blocks, like a box without peer access."""

    def __init__(self, rank, fail_on):
        self.rank, self.fail_on, self.calls = rank, fail_on, []

    def call(self, name, *arguments):
        import ctypes

        self.calls.append(name)
        if name == "tc_peer_block_bytes":
            arguments[3]._obj.value = 4096
        elif name == "tc_peer_block_create":
            arguments[2]._obj.value = 0x1000 * (self.rank + 1)
            ctypes.memmove(arguments[3], bytes([self.rank + 1]) * 64, 64)
        elif name == "tc_peer_block_open":
            if self.rank == self.fail_on:
                raise RuntimeError("tc_peer_block_open: peer access is not available (status 2)")
            arguments[2]._obj.value = 0x100000 + arguments[1][0]  # tagged with the owner's handle byte


class FakeDevice:
    index = 0


def peer_worker(rank, world, port, fail_on, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        library = FakePeerLibrary(rank, fail_on)
        original = torch.cuda.synchronize
        torch.cuda.synchronize = lambda device=None: None  # close() drains the device first; there is none here
        try:
            try:
                blocks = sharding.PeerBlocks(library, rank, world, 4, 8, FakeDevice())
            except RuntimeError as error:
                results[rank] = ("refused", str(error), list(library.calls))
                return
            table = [blocks.table[r] for r in range(world)]
            blocks.close()
            results[rank] = ("mapped", table, list(library.calls))
        finally:
            torch.cuda.synchronize = original
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fail_on", [None, 1])
def test_peer_blocks_are_mapped_by_all_ranks_or_by_none(fail_on):
    """Handles travel through one all-gather; if any rank cannot map a block, every rank gives the route
    up with the same error class, unmaps what it had mapped and frees its own block."""
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(peer_worker, args=(world, free_port(), fail_on, results), nprocs=world, join=True)
    assert set(results.keys()) == {0, 1}
    if fail_on is None:
        for rank in range(world):
            state, table, calls = results[rank]
            assert state == "mapped"
            assert table[rank] == 0x1000 * (rank + 1) and table[1 - rank] == 0x100000 + (2 - rank)
            assert calls == ["tc_peer_block_bytes", "tc_peer_block_create", "tc_peer_block_open",
                             "tc_peer_block_close", "tc_peer_block_destroy"]
    else:
        for rank in range(world):
            state, message, calls = results[rank]
            assert state == "refused" and message.startswith("peer exchange unavailable")
            assert calls[-1] == "tc_peer_block_destroy"
        assert "tc_peer_block_close" in results[0][2] and "tc_peer_block_close" not in results[1][2]


def absent_rank_worker(rank, world, port, results):
    import datetime

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    batch, capacity = 1, 64
    kcache, vcache, q, knew, vnew = oracle.seeded_normal(2, (batch, capacity, 8, 128), (batch, capacity, 8, 128),
                                                         (batch, 1, 32, 128), (batch, 1, 8, 128), (batch, 1, 8, 128))
    start, length = sharding.kv_sequence_shard(rank, world, capacity)
    driver = sharding.ShardedDecode(OracleOps(), rank, world, batch, capacity, torch.device("cpu"))
    out = torch.empty((batch, 1, 32, 128), dtype=torch.bfloat16)
    lse = torch.empty((batch, 32, 1), dtype=torch.float32)
    old = torch.tensor([40], dtype=torch.int32)
    if rank == 1:
        results[rank] = "left"
        return  # leaves between steps without joining the collective (its process then exits)
    try:
        driver.step(q, kcache[:, start:start + length].clone(), vcache[:, start:start + length].clone(), knew, vnew,
                    old, out, lse)
        results[rank] = "no error"
    except Exception as error:  # the collective ends with an error instead of hanging
        results[rank] = f"raised {type(error).__name__}"


def test_a_rank_that_never_joins_ends_the_step_with_an_error():
    """Failure on the host side, no GPU involved: one rank leaves before the exchange; the other rank's
    collective returns an error within the process-group timeout and the step raises."""
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(absent_rank_worker, args=(world, free_port(), results), nprocs=world, join=True)
    assert results[1] == "left"
    assert results[0].startswith("raised"), results[0]

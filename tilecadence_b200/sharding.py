"""Single-node multi-GPU drivers for the two shardable parts of the hot path.

The reference has no distributed code; these drivers implement the sharding the benchmark
configurations call for, one process per GPU with ``torch.distributed`` for the plumbing.

* Prefill shards by (batch, KV-head group): every unit is independent, so a rank simply runs the
  kernel on its slice of heads. No collective.
* Long-context decode shards the KV sequence: rank ``r`` keeps cache rows
  ``[r * shard, (r + 1) * shard)`` of every sequence, runs the split-KV kernel on them (the rank that
  owns row ``old_len`` performs the append), and produces a normalised partial O and a partial LSE.
  Two exchange routes merge them so that every rank ends with the full result:

  - ``exchange="nccl"``: one all-gather of the packed partials (``B*Hq*129`` floats per rank), then
    the LSE-weighted combine kernel. Three launches per step; the collective's latency dominates.
  - ``exchange="peer"``: one launch. The decode kernel itself stores the rank's partial into every
    rank's exchange block over NVLink (plain peer stores only; every 4-byte value travels with the
    call's epoch in the same 8-byte word, so no fence or separate flag is needed), polls its own block
    and merges in the same CTA. See ``tc_decode_exchange_out`` in the header.
"""
from __future__ import annotations

GROUP = 4
DIM = 128


def kv_head_slice(rank: int, world: int, kv_heads: int = 8):
    """Contiguous KV heads owned by ``rank`` and the matching query-head slice."""
    if kv_heads % world:
        raise ValueError(f"{kv_heads} KV heads do not divide over {world} ranks")
    per_rank = kv_heads // world
    kv = slice(rank * per_rank, (rank + 1) * per_rank)
    return kv, slice(kv.start * GROUP, kv.stop * GROUP)


def kv_sequence_shard(rank: int, world: int, capacity: int):
    """Global cache rows ``[start, start + length)`` owned by ``rank``."""
    if capacity % world:
        raise ValueError(f"capacity {capacity} does not divide over {world} ranks")
    length = capacity // world
    return rank * length, length


class PeerBlocks:
    """Every rank's exchange block of the fused decode exchange, mapped into this process.

    Construction is collective over ``group``: each rank creates its block on its own GPU, the
    64-byte interprocess handles travel through one all-gather, and each rank maps the others'
    blocks. ``table`` is the ``void*[world]`` array the C ABI takes. ``close`` is collective too.
    """

    def __init__(self, library, rank, world, batch, kv_heads, device, group=None):
        import ctypes

        import torch
        import torch.distributed as dist

        self.library, self.rank, self.world, self.device, self.group = library, rank, world, device, group
        size = ctypes.c_int64(0)
        library.call("tc_peer_block_bytes", batch, kv_heads, world, ctypes.byref(size))
        self.bytes = size.value
        own, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        library.call("tc_peer_block_create", device.index, self.bytes, ctypes.byref(own), handle)
        self.table = (ctypes.c_void_p * world)()
        self.table[rank] = own.value
        if world > 1:
            on_gpu = dist.get_backend(group) != "gloo"
            mine = torch.tensor(list(handle.raw), dtype=torch.uint8, device=device if on_gpu else "cpu")
            everyone = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(everyone, mine, group=group)
            failure = None
            for peer in range(world):
                if peer == rank:
                    continue
                mapped = ctypes.c_void_p()
                try:
                    library.call("tc_peer_block_open", device.index, bytes(everyone[peer].cpu().tolist()),
                                 ctypes.byref(mapped))
                except RuntimeError as error:  # keep going: the outcome must be agreed on by every rank
                    failure = failure or str(error)
                    continue
                self.table[peer] = mapped.value
            # Either every rank mapped every block or nobody uses the route.
            verdict = torch.tensor([0 if failure is None else 1], dtype=torch.uint8, device=mine.device)
            verdicts = [torch.empty_like(verdict) for _ in range(world)]
            dist.all_gather(verdicts, verdict, group=group)
            if any(int(v.item()) for v in verdicts):
                self.open = True
                self.close()
                raise RuntimeError("peer exchange unavailable: " + (failure or "another rank could not map the blocks"))
        self.open = True

    def close(self):
        import torch
        import torch.distributed as dist

        if not self.open:
            return
        self.open = False
        torch.cuda.synchronize(self.device)
        for peer in range(self.world):
            if peer != self.rank and self.table[peer]:
                self.library.call("tc_peer_block_close", self.device.index, self.table[peer])
        if self.world > 1:
            dist.barrier(group=self.group)  # nobody maps this rank's block any more
        self.library.call("tc_peer_block_destroy", self.device.index, self.table[self.rank])


class ShardedDecode:
    """Decode step over a KV-sequence-sharded cache.

    ``ops`` is the decode operator object of :mod:`tilecadence_b200.cuda_runtime`. Buffers are
    allocated once; ``step`` enqueues everything on the current stream and returns nothing, so the
    caller times it with events. ``group`` is the process group (default: world). ``exchange`` picks
    the route described in the module docstring; ``"peer"`` needs every rank on its own GPU of one
    node and makes construction collective (``close`` as well).
    """

    def __init__(self, ops, rank, world, batch, capacity, device, q_heads=32, group=None, exchange="nccl"):
        import torch

        if exchange not in ("nccl", "peer"):
            raise ValueError(f"unknown exchange route {exchange!r}")
        self.ops, self.rank, self.world, self.group = ops, rank, world, group
        self.batch, self.q_heads, self.exchange = batch, q_heads, exchange
        self.shard_start, self.shard_len = kv_sequence_shard(rank, world, capacity)
        self.rows = batch * q_heads
        self.packed_elems = self.rows * (DIM + 1)
        self.workspace = None
        self.peers = None
        if exchange == "peer":
            self.peers = PeerBlocks(ops.library, rank, world, batch, q_heads // GROUP, device, group)
            return
        self.packed = torch.empty(self.packed_elems, device=device, dtype=torch.float32)
        self.gathered = torch.empty((world, self.packed_elems), device=device, dtype=torch.float32)

    def close(self):
        if self.peers is not None:
            self.peers.close()

    def views(self, buffer):
        """(O [.., rows, 128], LSE [.., rows]) views of a packed buffer or of the gathered buffer."""
        split = self.rows * DIM
        if buffer.dim() == 1:
            return buffer[:split].view(self.rows, DIM), buffer[split:]
        return buffer[:, :split].unflatten(1, (self.rows, DIM)), buffer[:, split:]

    def step(self, q, kcache, vcache, knew, vnew, old_lengths, out, lse, num_splits=0, mapping=1):
        import torch
        import torch.distributed as dist

        if kcache.size(1) != self.shard_len:
            raise RuntimeError(f"rank {self.rank} expects a cache shard of {self.shard_len} rows")
        if self.workspace is None:
            spec = self.ops.workspace_spec(q, kcache, old_lengths, num_splits, mapping, True)
            self.workspace = tuple(torch.empty(n, device=q.device, dtype=torch.float32) for n in spec[1:3])
        if self.peers is not None:
            self.ops.exchange_out(q, kcache, vcache, knew, vnew, old_lengths, out, lse, *self.workspace, num_splits,
                                  mapping, True, self.shard_start, self.rank, self.peers.table, self.peers.bytes)
            return
        partial_o, partial_lse = self.views(self.packed)
        self.ops.partial_out(q, kcache, vcache, knew, vnew, old_lengths, partial_o, partial_lse, *self.workspace,
                             num_splits, mapping, True, self.shard_start)
        if self.world > 1:
            if dist.get_backend(self.group) == "gloo":
                dist.all_gather(list(self.gathered.unbind(0)), self.packed, group=self.group)
            else:
                dist.all_gather_into_tensor(self.gathered, self.packed, group=self.group)
        else:
            self.gathered[0].copy_(self.packed)
        gathered_o, gathered_lse = self.views(self.gathered)
        self.ops.combine_partials(gathered_o, gathered_lse, out, lse)

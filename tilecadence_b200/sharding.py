"""Single-node multi-GPU drivers for the two shardable parts of the hot path.

The reference has no distributed code; these drivers implement the sharding the benchmark
configurations call for, one process per GPU with ``torch.distributed`` for the plumbing.

* Prefill shards by (batch, KV-head group): every unit is independent, so a rank simply runs the
  kernel on its slice of heads. No collective.
* Long-context decode shards the KV sequence: rank ``r`` keeps cache rows
  ``[r * shard, (r + 1) * shard)`` of every sequence, runs the split-KV kernel on them (the rank that
  owns row ``old_len`` performs the append), and produces a normalised partial O and a partial LSE.
  One all-gather moves the packed partials (``B*Hq*129`` floats per rank) to every rank and the
  LSE-weighted combine kernel merges them, so every rank ends with the full result. Nothing reads
  another GPU's memory directly.
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


class ShardedDecode:
    """Decode step over a KV-sequence-sharded cache: kernel -> all-gather -> combine.

    ``ops`` is the decode operator object of :mod:`tilecadence_b200.cuda_runtime`. Buffers are
    allocated once; ``step`` enqueues everything on the current stream and returns nothing, so the
    caller times it with events. ``group`` is the process group (default: world).
    """

    def __init__(self, ops, rank, world, batch, capacity, device, q_heads=32, group=None):
        import torch

        self.ops, self.rank, self.world, self.group = ops, rank, world, group
        self.batch, self.q_heads = batch, q_heads
        self.shard_start, self.shard_len = kv_sequence_shard(rank, world, capacity)
        self.rows = batch * q_heads
        self.packed_elems = self.rows * (DIM + 1)
        self.packed = torch.empty(self.packed_elems, device=device, dtype=torch.float32)
        self.gathered = torch.empty((world, self.packed_elems), device=device, dtype=torch.float32)
        self.workspace = None

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

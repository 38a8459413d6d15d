"""How the path spreads over the GPUs of one box (one process per GPU).

Two ways, both new design (the reference has no multi-GPU mode):

* by sequence — independent units; a rank owns the page pool, block tables and
  prefix cache of its sequences, and a session always lands on the same rank
  (hash of the session root); no collective on the data path;
* by KV-head group for one long sequence — rank g holds the pages of kv heads
  [g*KV/G, (g+1)*KV/G) and computes the Q/G query heads of those groups; the only
  exchange is the attention output row of a layer, which every rank needs whole. On GPUs
  the attention launch itself stores its slice into the peers' rows and trades flags with
  them (Batch.enqueue_step_exchange over memory mapped with peer_export / peer_open); an
  all-gather of torch.distributed (NCCL; gloo in the CPU tests) does the same in a separate
  call and is what the CPU tests of the split use.
"""
from __future__ import annotations

from dataclasses import dataclass


def sequences_of_rank(n_sequences: int, world: int, rank: int) -> range:
    """Contiguous, balanced split of sequence indices (sizes differ by at most one)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world {world}")
    base, extra = divmod(n_sequences, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def rank_of_session(session_root: bytes, world: int) -> int:
    """A session's blocks stay on one GPU: rank = first 8 bytes of its root hash mod world."""
    if len(session_root) != 32:
        raise ValueError("session root must be a 32-byte block hash")
    return int.from_bytes(session_root[:8], "little") % world


@dataclass(frozen=True)
class HeadShard:
    kv_head_start: int
    kv_heads: int
    q_head_start: int
    q_heads: int

    def q_slice(self, head_dim: int) -> slice:
        return slice(self.q_head_start * head_dim, (self.q_head_start + self.q_heads) * head_dim)

    def kv_slice(self, head_dim: int) -> slice:
        return slice(self.kv_head_start * head_dim, (self.kv_head_start + self.kv_heads) * head_dim)


def head_shard(q_heads: int, kv_heads: int, world: int, rank: int) -> HeadShard:
    """KV heads are the unit: at most kv_heads ranks, and kv_heads must divide evenly."""
    if q_heads % kv_heads != 0:
        raise ValueError(f"invalid GQA: q_heads={q_heads} is not a multiple of kv_heads={kv_heads}")
    if world > kv_heads or kv_heads % world != 0:
        raise ValueError(f"cannot shard {kv_heads} kv heads over {world} ranks")
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world {world}")
    per = kv_heads // world
    gqa = q_heads // kv_heads
    return HeadShard(rank * per, per, rank * per * gqa, per * gqa)


def all_gather_heads(local_out, group=None):
    """All-gather of per-rank attention outputs [.., q_heads_local*head_dim] along the last
    dimension into [.., q_heads*head_dim] (rank order = head order)."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    flat = local_out.contiguous()
    parts = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(parts, flat, group=group)
    return torch.cat(parts, dim=-1)

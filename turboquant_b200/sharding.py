"""Multi-GPU partition of the decode path and the one collective it needs.

The attention path shards by (sequence, kv head) with no exchange step: a rank
needs only its own compressed records and the query heads of its kv heads.
With R ranks and H kv heads the heads are split first (as vLLM tensor
parallelism does, reference integration/vllm.py:361-372 hooks the worker's
local heads); once every rank owns a single head, the sequences of that head
are split among the ranks that share it.  The only collective is an all-gather
of the per-rank output slabs (batch, local query heads, D) when a caller wants
the full (batch, all query heads, D) tensor on every rank.

One process per GPU; `torch.distributed` (NCCL on GPUs, gloo in CPU tests)
does the plumbing.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Shard:
    """What one rank owns: kv heads [head0, head1) for sequences [seq0, seq1)."""
    rank: int
    world_size: int
    head0: int
    head1: int
    seq0: int
    seq1: int

    @property
    def num_heads(self) -> int:
        return self.head1 - self.head0

    @property
    def num_seqs(self) -> int:
        return self.seq1 - self.seq0

    def query_heads(self, group: int) -> range:
        """Query heads of this shard when `group` query heads share a kv head."""
        return range(self.head0 * group, self.head1 * group)


def partition(num_seqs: int, num_kv_heads: int, world_size: int, rank: int) -> Shard:
    """Heads first, then sequences.  Every (sequence, head) pair has exactly one owner."""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of {world_size}")
    head_ways = min(world_size, num_kv_heads)
    if num_kv_heads % head_ways != 0 or world_size % head_ways != 0:
        raise ValueError(f"{num_kv_heads} kv heads do not split over {world_size} ranks")
    seq_ways = world_size // head_ways
    hpr = num_kv_heads // head_ways
    head_slot, seq_slot = rank // seq_ways, rank % seq_ways
    seq0 = num_seqs * seq_slot // seq_ways
    seq1 = num_seqs * (seq_slot + 1) // seq_ways
    return Shard(rank, world_size, head_slot * hpr, (head_slot + 1) * hpr, seq0, seq1)


def gather_head_outputs(local_out: torch.Tensor, shard: Shard, num_seqs: int, num_kv_heads: int,
                        group=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-gather the ranks' output slabs into (num_seqs, all query heads, D) on every rank.

    local_out: (shard.num_seqs, shard.num_heads * G, D).  Slabs travel in rank
    order and are placed by each rank's Shard, so ragged sequence splits work.
    """
    world = shard.world_size
    g_heads = local_out.shape[1] // shard.num_heads
    d = local_out.shape[2]
    if out is None:
        out = torch.empty(num_seqs, num_kv_heads * g_heads, d, dtype=local_out.dtype, device=local_out.device)
    if world == 1:
        out.copy_(local_out)
        return out
    shards = [partition(num_seqs, num_kv_heads, world, r) for r in range(world)]
    rows = shards[0].num_seqs
    if all(s.num_seqs == rows for s in shards):
        # even split (the usual case): gather straight from the caller's slab and place all slabs
        # with one strided copy - rank = head_slot * seq_ways + seq_slot
        head_ways = min(world, num_kv_heads)
        seq_ways = world // head_ways
        hg = local_out.shape[1]
        flat = _gather_buffer((world, rows, hg, d), local_out.dtype, local_out.device)
        dist.all_gather_into_tensor(flat.view(world * rows, hg, d), local_out.contiguous(), group=group)
        out.view(seq_ways, rows, head_ways, hg, d).copy_(flat.view(head_ways, seq_ways, rows, hg, d).permute(1, 2, 0, 3, 4))
        return out
    max_rows = max(s.num_seqs for s in shards)
    send = torch.zeros(max_rows, local_out.shape[1], d, dtype=local_out.dtype, device=local_out.device)
    send[: shard.num_seqs].copy_(local_out)
    flat = torch.empty(world * max_rows, *send.shape[1:], dtype=send.dtype, device=send.device)
    dist.all_gather_into_tensor(flat, send, group=group)    # rank r's slab is rows [r*max_rows, (r+1)*max_rows)
    recv = flat.view(world, *send.shape)
    for s in shards:
        out[s.seq0:s.seq1, s.head0 * g_heads:s.head1 * g_heads].copy_(recv[s.rank, : s.num_seqs])
    return out


_GATHER_BUFFERS: dict = {}


def _gather_buffer(shape, dtype, device) -> torch.Tensor:
    """Receive buffer of the all-gather, kept between calls (one per shape)."""
    key = (tuple(shape), dtype, str(device))
    buf = _GATHER_BUFFERS.get(key)
    if buf is None:
        buf = _GATHER_BUFFERS[key] = torch.empty(shape, dtype=dtype, device=device)
    return buf


def reduce_timing(local_ms: float, local_units: float, device, group=None) -> tuple[float, float]:
    """(max over ranks of the time, sum over ranks of the units processed)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return local_ms, local_units
    t = torch.tensor([local_ms], dtype=torch.float64, device=device)
    u = torch.tensor([local_units], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    dist.all_reduce(u, op=dist.ReduceOp.SUM, group=group)
    return float(t.item()), float(u.item())

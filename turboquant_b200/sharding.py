"""Multi-GPU partition of the decode path and the one collective it needs.

The attention path shards by (sequence, kv head) with no exchange step: a rank
needs only its own compressed records and the query heads of its kv heads.
With R ranks the SEQUENCES are split first: a rank then owns a band of whole
rows of the (sequences, query heads, D) output, the decode kernel writes
straight into that band of the full tensor and the all-gather lands every
other rank's band in place - no staging copy on either side.  Only when there
are more ranks than sequences are the kv heads of a sequence band split as
well (the reference hooks each tensor-parallel worker's local heads,
integration/vllm.py:361-372).  The only collective is the all-gather of the
per-rank output slabs when a caller wants the full tensor on every rank.

One process per GPU; `torch.distributed` (NCCL on GPUs, gloo in CPU tests)
does the plumbing.
"""

from __future__ import annotations

from dataclasses import dataclass
from functools import lru_cache
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


@lru_cache(maxsize=None)
def _ways(num_seqs: int, num_kv_heads: int, world_size: int) -> tuple[int, int]:
    """(sequence ways, head ways): as many sequence bands as divide the world and do not exceed
    the sequences; the remaining factor splits the kv heads."""
    seq_ways = max(w for w in range(1, world_size + 1) if world_size % w == 0 and w <= max(1, num_seqs))
    head_ways = world_size // seq_ways
    if num_kv_heads % head_ways != 0:
        raise ValueError(f"{num_seqs} sequences x {num_kv_heads} kv heads do not split over {world_size} ranks")
    return seq_ways, head_ways


@lru_cache(maxsize=None)
def partition(num_seqs: int, num_kv_heads: int, world_size: int, rank: int) -> Shard:
    """Sequences first, then heads.  Every (sequence, head) pair has exactly one owner;
    rank = sequence band * head ways + head slot."""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of {world_size}")
    seq_ways, head_ways = _ways(num_seqs, num_kv_heads, world_size)
    hpr = num_kv_heads // head_ways
    seq_slot, head_slot = rank // head_ways, rank % head_ways
    seq0 = num_seqs * seq_slot // seq_ways
    seq1 = num_seqs * (seq_slot + 1) // seq_ways
    return Shard(rank, world_size, head_slot * hpr, (head_slot + 1) * hpr, seq0, seq1)


@lru_cache(maxsize=None)
def _all_shards(num_seqs: int, num_kv_heads: int, world: int) -> tuple:
    return tuple(partition(num_seqs, num_kv_heads, world, r) for r in range(world))


@lru_cache(maxsize=None)
def _whole_row_bands(num_seqs: int, num_kv_heads: int, world: int) -> bool:
    shards = _all_shards(num_seqs, num_kv_heads, world)
    return all(s.num_seqs == shards[0].num_seqs and s.num_heads == num_kv_heads for s in shards)


def output_slab(out_full: torch.Tensor, shard: Shard, num_kv_heads: int) -> Optional[torch.Tensor]:
    """The rows of the full (sequences, query heads, D) output this rank produces, as a view the
    decode kernel can write into, when the shard is a band of whole rows and the bands of all ranks
    are equally high (then `gather_head_outputs` works in place); None otherwise."""
    if shard.num_heads != num_kv_heads or shard.num_seqs * shard.world_size != out_full.shape[0]:
        return None
    return out_full[shard.seq0:shard.seq1]


def gather_head_outputs(local_out: torch.Tensor, shard: Shard, num_seqs: int, num_kv_heads: int,
                        group=None, out: Optional[torch.Tensor] = None, async_op: bool = False):
    """All-gather the ranks' output slabs into (num_seqs, all query heads, D) on every rank.

    local_out: (shard.num_seqs, shard.num_heads * G, D).  When every rank owns an equally high band
    of whole rows, the collective writes straight into `out`; if `local_out` already is this rank's
    band of `out` (see `output_slab`) nothing is copied at all.  Other partitions (ragged sequence
    splits, split heads) go through a padded receive buffer and are placed by each rank's Shard.
    Returns `out`, or (out, work handle) with async_op=True.
    """
    world = shard.world_size
    g_heads = local_out.shape[1] // shard.num_heads
    d = local_out.shape[2]
    if out is None:
        out = torch.empty(num_seqs, num_kv_heads * g_heads, d, dtype=local_out.dtype, device=local_out.device)
    in_place = local_out.data_ptr() == out[shard.seq0:shard.seq1].data_ptr() and shard.num_heads == num_kv_heads
    if world == 1:
        if not in_place:
            out.copy_(local_out)
        return (out, None) if async_op else out
    shards = _all_shards(num_seqs, num_kv_heads, world)
    rows = shards[0].num_seqs
    if _whole_row_bands(num_seqs, num_kv_heads, world):
        # bands of whole rows in rank order: the gathered tensor IS the output
        work = dist.all_gather_into_tensor(out, local_out if in_place else local_out.contiguous(), group=group,
                                           async_op=async_op)
        return (out, work) if async_op else out
    max_rows = max(s.num_seqs for s in shards)
    send = torch.zeros(max_rows, local_out.shape[1], d, dtype=local_out.dtype, device=local_out.device)
    send[: shard.num_seqs].copy_(local_out)
    flat = _gather_buffer((world * max_rows, *send.shape[1:]), send.dtype, send.device)
    dist.all_gather_into_tensor(flat, send, group=group)    # rank r's slab is rows [r*max_rows, (r+1)*max_rows)
    recv = flat.view(world, *send.shape)
    for s in shards:
        out[s.seq0:s.seq1, s.head0 * g_heads:s.head1 * g_heads].copy_(recv[s.rank, : s.num_seqs])
    return (out, None) if async_op else out


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

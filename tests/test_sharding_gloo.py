"""Multi-rank host logic on CPU: 2 gloo ranks (and single-process checks of the
partition rule).  No GPU: the compute on each rank is a stand-in."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from turboquant_b200.sharding import gather_head_outputs, output_slab, partition, reduce_timing


@pytest.mark.parametrize("seqs,heads,world", [(256, 8, 1), (256, 8, 2), (256, 8, 4), (256, 8, 8), (64, 8, 16),
                                              (5, 4, 8), (7, 2, 2), (1, 4, 4)])
def test_partition_covers_every_pair_once(seqs, heads, world):
    owner = torch.zeros(seqs, heads, dtype=torch.int32)
    for r in range(world):
        s = partition(seqs, heads, world, r)
        owner[s.seq0:s.seq1, s.head0:s.head1] += 1
        assert list(s.query_heads(4)) == list(range(s.head0 * 4, s.head1 * 4))
    assert bool((owner == 1).all())


def test_partition_is_sequences_first():
    """With enough sequences every rank owns whole output rows (all kv heads of a band of sequences);
    heads are split only when the ranks outnumber the sequences."""
    for world in (1, 2, 4, 8):
        for r in range(world):
            s = partition(256, 8, world, r)
            assert (s.head0, s.head1) == (0, 8) and (s.seq0, s.seq1) == (256 * r // world, 256 * (r + 1) // world)
    s = partition(1, 4, 4, 2)
    assert (s.seq0, s.seq1, s.head0, s.head1) == (0, 1, 2, 3)
    s = partition(2, 8, 8, 5)      # 2 sequence bands x 4 head slots
    assert (s.seq0, s.seq1, s.head0, s.head1) == (1, 2, 2, 4)


def test_partition_rejects_bad_worlds():
    with pytest.raises(ValueError):
        partition(1, 8, 3, 0)      # three head slots do not divide eight heads
    with pytest.raises(ValueError):
        partition(8, 8, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, seqs, heads, g, d, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        shard = partition(seqs, heads, world, rank)
        # stand-in for the decode output: value encodes (sequence, query head)
        seq = torch.arange(shard.seq0, shard.seq1).view(-1, 1, 1).float()
        qh = torch.arange(shard.head0 * g, shard.head1 * g).view(1, -1, 1).float()
        local = (seq * 1000 + qh).expand(-1, -1, d).contiguous()
        full = gather_head_outputs(local, shard, seqs, heads)
        want = (torch.arange(seqs).view(-1, 1, 1) * 1000 + torch.arange(heads * g).view(1, -1, 1)).float().expand(-1, -1, d)
        ok = torch.equal(full, want)
        # in place: the rank writes its band of the full tensor, the gather fills in the others
        buf = torch.full((seqs, heads * g, d), -1.0)
        slab = output_slab(buf, shard, heads)
        if seqs % world == 0 and shard.num_heads == heads:
            slab.copy_(local)
            full2, work = gather_head_outputs(slab, shard, seqs, heads, out=buf, async_op=True)
            work.wait()
            ok = ok and full2.data_ptr() == buf.data_ptr() and torch.equal(buf, want)
        else:
            ok = ok and slab is None
        ms, units = reduce_timing(10.0 + rank, 100.0 * (rank + 1), "cpu")
        ok = ok and ms == 10.0 + world - 1 and units == 100.0 * world * (world + 1) / 2
        result[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("seqs,heads", [(6, 2), (5, 1), (1, 2)])
def test_two_gloo_ranks_gather_and_time(seqs, heads):
    world = 2
    with mp.Manager() as mgr:
        result = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), seqs, heads, 4, 8, result), nprocs=world, join=True)
        assert dict(result) == {0: True, 1: True}

"""tq_decode_static: decode for hosts that may not allocate device memory.

A serving engine usually grabs nearly all HBM for its KV pool at start-up and
may lock its allocator afterwards; a plugin called from inside it then has no
way to obtain the scratch buffer tq_decode wants.  tq_decode_static keeps that
scratch in a fixed array inside the library instead.  These tests call it
through the C ABI twice in a row with a call of another shape in between (the
array keeps the earlier calls' contents, and the in-between call leaves its
partial results where the next call's tickets live, so the clearing is really
needed), compare with tq_decode on the same inputs (same kernels: results must
agree to the tolerance the other decode tests use) and with the CPU oracle,
read the array's status word, and check that the free device memory is the
same before and after a call made with a preallocated output.  A launch that
cannot fit the array must be refused with a clear error, not run.

Collected last on purpose: a run that stops at the first failure has then
already executed every other test.
"""

import ctypes as C

import pytest
import torch

from oracle import tq_oracle as O

pytestmark = pytest.mark.gpu


def _setup(dev, d, h, qh, n, ring):
    from turboquant_b200 import _engine as E
    c = E.LayerConstants(d, 3, 2, dev, seed=63)
    k, v = O.synth_kv(n + ring, h, d, seed=17, dtype=torch.bfloat16)
    pool = E.BlockPool(c, h, E.blocks_for(n))
    bt = E.identity_block_table(pool.num_blocks, dev)
    E.store(c, pool, k[:n].to(dev), v[:n].to(dev), stride_token=h * d, stride_head=d, n_tokens=n, n_heads=h,
            block_table=bt, start_pos=0)
    rk, rv = k[n:].to(dev).contiguous(), v[n:].to(dev).contiguous()
    return E, c, pool, bt, rk, rv, k, v


def _static_status(dev) -> int:
    from turboquant_b200 import _lib
    out = C.c_int32(-99)
    rc = _lib.lib().tq_decode_static_read_status(torch.cuda.current_stream(dev).cuda_stream, C.byref(out))
    assert rc == 0
    return out.value


@pytest.mark.parametrize("d,h,qh", [(256, 4, 16), (128, 8, 32)])
def test_static_scratch_decode_matches_workspace_decode(d, h, qh):
    dev = torch.device("cuda:0")
    n, ring = 2100, 40
    E, c, pool, bt, rk, rv, k, v = _setup(dev, d, h, qh, n, ring)
    lens = torch.tensor([n, n - 500], dtype=torch.int32, device=dev)
    rl = torch.tensor([ring, 7], dtype=torch.int32, device=dev)
    bt2 = bt.unsqueeze(0).expand(2, -1).contiguous()
    kw = dict(ring_k=rk, ring_v=rv, ring_lens=rl, max_ring_len=ring, ring_stride_seq=0, ring_stride_token=h * d,
              num_splits=6)
    ws = E.Workspace(dev)
    out = torch.empty(2, qh, d, dtype=torch.bfloat16, device=dev)
    assert _static_status(dev) == 0           # also the set-up call: looks up the array's address
    ost = O.OracleStore(d, h, 3, 2, c.centroids_cpu, c.boundaries_cpu, pi=c.Pi.cpu(), s=c.S.cpu())
    ost.append_chunk(k[:n], v[:n])
    for call in range(2):   # two calls in a row: the second one meets what came before it
        q = O.synth_query(2, qh, d, seed=100 + call, dtype=torch.bfloat16).to(dev)
        ref = E.decode(c, pool, ws, q, bt2, lens, n, **kw).float()
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0]
        got = E.decode(c, pool, None, q, bt2, lens, n, static_scratch=True, out=out, **kw)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info(dev)[0] == free_before     # nothing was allocated on the device
        assert got.data_ptr() == out.data_ptr()
        got = got.float()
        assert _static_status(dev) == 0
        assert torch.isfinite(got).all()
        torch.testing.assert_close(got, ref, rtol=3e-2, atol=3e-3)
        cos = torch.nn.functional.cosine_similarity(got.flatten().double(), ref.flatten().double(), dim=0)
        assert float(cos) >= 0.9999
        # sequence 0 (full length, full ring) against the CPU oracle
        want = O.hybrid_attention(q[:1].cpu(), ost.get_flat_cache(), k[n:], v[n:], h, c.Pi.cpu(), c.S.cpu(),
                                  c.centroids_cpu)
        cos = torch.nn.functional.cosine_similarity(got[:1].cpu().flatten().double(), want.flatten().double(), dim=0)
        assert float(cos) >= 0.9999
        # a call of another shape in between: one sequence, many splits - its partial results land
        # where the two-sequence call keeps its tickets and prepared query
        E.decode(c, pool, None, q[:1], bt2[:1], lens[:1], n, static_scratch=True, num_splits=24)
        torch.cuda.synchronize()
        assert _static_status(dev) == 0


def test_static_scratch_refuses_oversized_launch():
    from turboquant_b200 import _lib
    dev = torch.device("cuda:0")
    d, h, qh, n = 128, 8, 32, 256
    E, c, pool, bt, rk, rv, _, _ = _setup(dev, d, h, qh, n, 0)
    assert _lib.lib().tq_decode_static_scratch_bytes() == 8 << 20
    batch = 2048                                  # partials alone need far more than 8 MiB
    q = torch.zeros(batch, qh, d, dtype=torch.bfloat16, device=dev)
    lens = torch.full((batch,), n, dtype=torch.int32, device=dev)
    bt2 = bt.unsqueeze(0).expand(batch, -1).contiguous()
    with pytest.raises(_lib.TQError) as err:
        E.decode(c, pool, None, q, bt2, lens, n, static_scratch=True, num_splits=1)
    assert err.value.status == -6 and "scratch" in str(err.value)
    assert _static_status(dev) == 0               # a refused call enqueues nothing and reports nothing

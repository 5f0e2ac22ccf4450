"""tq_decode_static: decode for hosts that may not allocate device memory.

A serving engine usually grabs nearly all HBM for its KV pool at start-up and
may lock its allocator afterwards; a plugin called from inside it then has no
way to obtain the scratch buffer tq_decode wants.  tq_decode_static keeps that
scratch in a fixed array inside the library instead.  This test calls it
through the C ABI twice in a row (the array keeps the first call's contents, so
the second call proves the re-zeroing) and compares with tq_decode on the same
inputs; both run the same kernels, so the results must agree to the tolerance
the other decode tests use.  It also checks that a launch that cannot fit the
array is refused with a clear error rather than run.

Collected last on purpose: a run that stops at the first failure has then
already executed every other test.
"""

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
    return E, c, pool, bt, rk, rv


@pytest.mark.parametrize("d,h,qh", [(256, 4, 16), (128, 8, 32)])
def test_static_scratch_decode_matches_workspace_decode(d, h, qh):
    dev = torch.device("cuda:0")
    n, ring = 2100, 40
    E, c, pool, bt, rk, rv = _setup(dev, d, h, qh, n, ring)
    lens = torch.tensor([n, n - 500], dtype=torch.int32, device=dev)
    rl = torch.tensor([ring, 7], dtype=torch.int32, device=dev)
    bt2 = bt.unsqueeze(0).expand(2, -1).contiguous()
    kw = dict(ring_k=rk, ring_v=rv, ring_lens=rl, max_ring_len=ring, ring_stride_seq=0, ring_stride_token=h * d,
              num_splits=6)
    ws = E.Workspace(dev)
    for call in range(2):   # two calls in a row: the second one meets the first one's leftovers
        q = O.synth_query(2, qh, d, seed=100 + call, dtype=torch.bfloat16).to(dev)
        ref = E.decode(c, pool, ws, q, bt2, lens, n, **kw).float()
        got = E.decode(c, pool, None, q, bt2, lens, n, static_scratch=True, **kw).float()
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        torch.testing.assert_close(got, ref, rtol=3e-2, atol=3e-3)
        cos = torch.nn.functional.cosine_similarity(got.flatten().double(), ref.flatten().double(), dim=0)
        assert float(cos) >= 0.9999


def test_static_scratch_refuses_oversized_launch():
    from turboquant_b200 import _lib
    dev = torch.device("cuda:0")
    d, h, qh, n = 128, 8, 32, 256
    E, c, pool, bt, rk, rv = _setup(dev, d, h, qh, n, 0)
    assert _lib.lib().tq_decode_static_scratch_bytes() == 8 << 20
    batch = 2048                                  # partials alone need far more than 8 MiB
    q = torch.zeros(batch, qh, d, dtype=torch.bfloat16, device=dev)
    lens = torch.full((batch,), n, dtype=torch.int32, device=dev)
    bt2 = bt.unsqueeze(0).expand(batch, -1).contiguous()
    with pytest.raises(_lib.TQError) as err:
        E.decode(c, pool, None, q, bt2, lens, n, static_scratch=True, num_splits=1)
    assert err.value.status == -6 and "scratch" in str(err.value)

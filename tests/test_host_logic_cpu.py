"""Host-side logic that needs no GPU: the ring buffer's drain policy (reference
capture.py:21-120), the split planner and the sharding arithmetic."""

import pytest
import torch

from turboquant_b200 import _engine as E
from turboquant_b200.capture import RingBuffer


def _tok(i, h=2, d=4):
    return torch.full((1, h, d), float(i))


def test_ring_buffer_drains_whole_buffer_when_the_next_token_arrives():
    rb = RingBuffer(4, 2, 4, "cpu", torch.float32)
    assert rb.peek() is None and rb.drain() is None and rb.size == 0
    for i in range(4):
        assert rb.write(_tok(i), _tok(10 + i), 1) is None
    assert rb.is_full and rb.size == 4
    k, v = rb.peek()
    assert [float(x) for x in k[:, 0, 0]] == [0, 1, 2, 3] and float(v[3, 0, 0]) == 13
    out = rb.write(_tok(4), _tok(14), 1)              # the fifth token pushes the four out, as one chunk
    assert out is not None and out[0].shape == (4, 2, 4)
    assert [float(x) for x in out[0][:, 0, 0]] == [0, 1, 2, 3]
    assert rb.size == 1 and rb.total_written == 5
    k, _ = rb.peek()
    assert float(k[0, 0, 0]) == 4


def test_ring_buffer_long_write_drains_every_full_buffer():
    rb = RingBuffer(4, 1, 2, "cpu", torch.float32)
    keys = torch.arange(11, dtype=torch.float32).view(11, 1, 1).expand(11, 1, 2).contiguous()
    out = rb.write(keys, keys, 11)
    # 11 tokens through a 4-token ring: two full buffers leave, three tokens stay
    assert out is not None and out[0].shape[0] == 8
    assert [float(x) for x in out[0][:, 0, 0]] == list(range(8))
    assert rb.size == 3 and [float(x) for x in rb.peek()[0][:, 0, 0]] == [8, 9, 10]
    k, v = rb.drain()
    assert k.shape[0] == 3 and rb.size == 0 and rb.peek() is None
    rb.reset()
    assert rb.total_written == 0


@pytest.mark.parametrize("batch,h,n,ring", [(1, 4, 32768, 128), (1, 4, 32768, 0), (64, 8, 32768, 0), (256, 8, 8192, 0),
                                            (1, 8, 1 << 20, 100), (2, 2, 100, 16), (1, 1, 16, 0), (1, 4, 0, 40)])
def test_split_planner_keeps_the_kernels_limits(batch, h, n, ring):
    sms = 148
    s = E.choose_splits(batch, h, n, sms, ring)
    nblk = (n + 15) // 16
    assert s >= 1
    # the tensor-core kernel keeps a split's block-table slice in shared memory: at most 1024 entries
    assert -(-nblk // s) + 1 <= 1024
    # with few (sequence, head) pairs and a history that does not need more CTAs than there are SMs (a CTA
    # takes at most 512 records) the launch is one wave: history CTAs + ring CTAs of 64 tokens <= SMs
    ring_ctas = (ring + 63) // 64
    if -(-nblk // 512) <= sms // (batch * h) - ring_ctas and nblk >= 12 * s:
        assert batch * h * (s + ring_ctas) <= sms


def test_config1_split_is_five_record_rounds_per_warp():
    s = E.choose_splits(1, 4, 32768, 148, 128)
    assert s == 35                                    # 37 slots per head: 35 history + 2 ring CTAs
    assert -(-2048 // s) <= 5 * 12                    # at most five records per warp of a 12-warp CTA


@pytest.mark.parametrize("d,bits", [(128, 2), (128, 3), (256, 2), (256, 3), (64, 4), (576, 3)])
def test_own_lloyd_max_solver_reproduces_the_shipped_code_books(d, bits):
    """The package's solver (closed-form cell integrals) against the JSON files the kernels use, which
    came from the reference's quadrature-based solver (codebook.py:68-143): same starting point and
    stopping rule, so the same centroids and boundaries to well below 1e-6."""
    import json
    import os
    import numpy as np
    from turboquant_b200 import codebook as CB
    with open(os.path.join(CB._CODEBOOK_DIR, f"codebook_d{d}_b{bits}.json")) as fh:
        shipped = json.load(fh)
    own = CB.compute_lloyd_max_codebook(d, bits)
    assert len(own["centroids"]) == 2 ** bits and len(own["boundaries"]) == 2 ** bits + 1
    assert np.abs(np.array(own["centroids"]) - np.array(shipped["centroids"])).max() <= 1e-6
    assert np.abs(np.array(own["boundaries"]) - np.array(shipped["boundaries"])).max() <= 1e-6
    assert abs(own["mse_per_coord"] - shipped["mse_per_coord"]) <= 1e-9
    assert own["boundaries"][0] == -1.0 and own["boundaries"][-1] == 1.0


def test_compressed_cache_spec_page_arithmetic():
    """Page geometry an engine sizes its block pool with: bytes per page = 16 tokens x kv heads x the
    reference's per-token accounting (store.py:116-128), against bf16 K+V pages of the same block."""
    from turboquant_b200.paged_cache import CompressedCacheSpec
    s = CompressedCacheSpec(128, 8, 3, 2)
    assert (s.bytes_per_token, s.page_size_bytes, s.bf16_page_size_bytes) == (100, 12800, 65536)
    assert CompressedCacheSpec(256, 4, 3, 2).bytes_per_token == 196
    assert CompressedCacheSpec(128, 8, 4, 4).bytes_per_token == 164
    assert s.num_blocks_for(10 ** 9) == 78125 and s.max_memory_usage_bytes(32768 + 5) == 2049 * 12800
    with pytest.raises(ValueError):
        CompressedCacheSpec(128, 8, 3, 2, block_size=32)

"""Decode attention over compressed history plus the exact recent tokens
(reference score.py:29-173).

The reference dequantises the whole history to fp32 and runs einsum / softmax /
einsum.  Here one fused kernel streams the packed records, scores them against
the rotated query, keeps an online softmax jointly with the exact ring tokens
and accumulates the dequantised values; nothing is materialised.
"""

from __future__ import annotations

import logging
import math
from typing import Optional

import torch

from . import _engine as E
from .store import CompressedKVStore

logger = logging.getLogger("turboquant.score")

MIN_HISTORY_FOR_TQ = 16


def compute_hybrid_attention(query: torch.Tensor, store: CompressedKVStore, recent_k: Optional[torch.Tensor],
                             recent_v: Optional[torch.Tensor], num_query_heads: int,
                             scale: Optional[float] = None) -> torch.Tensor:
    """query (T, Qh, D); recent_k / recent_v (R, H, D) or None -> (T, Qh, D).

    Every query token attends to all history and all recent tokens (no causal
    mask, as in the reference); history shorter than 16 tokens is ignored.
    """
    E.require_cuda(query, "query")
    t, qh, d = query.shape
    if qh != num_query_heads or d != store.head_dim:
        raise ValueError(f"query shape {tuple(query.shape)} does not match {num_query_heads} heads x {store.head_dim}")
    if num_query_heads % store.num_kv_heads != 0:
        raise ValueError(f"Incompatible GQA shapes: Q={qh}, H_kv={store.num_kv_heads}")
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    n = store.num_tokens
    r = 0 if recent_k is None else int(recent_k.shape[0])
    if (n < MIN_HISTORY_FOR_TQ) and r == 0:
        return torch.zeros(t, qh, d, device=query.device, dtype=query.dtype)

    dev = query.device
    seq_lens = store.seq_len_device if t == 1 else store.seq_len_device.expand(t).contiguous()
    bt = store.block_table if t == 1 else store.block_table.unsqueeze(0).expand(t, -1).contiguous()
    kwargs = {}
    if r > 0:
        if recent_k.stride(2) != 1 or recent_k.stride(1) != d or recent_v.stride() != recent_k.stride():
            recent_k, recent_v = recent_k.contiguous(), recent_v.contiguous()
        kwargs = dict(ring_k=recent_k, ring_v=recent_v,
                      ring_lens=E.const_i32(dev, r, t), max_ring_len=r,
                      ring_stride_seq=0, ring_stride_token=recent_k.stride(0))
    return E.decode(store.consts, store.pool, store.workspace, query, bt, seq_lens, n, scale=scale,
                    min_history=MIN_HISTORY_FOR_TQ, **kwargs)

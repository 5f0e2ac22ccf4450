"""A compressed paged KV cache that the serving engine allocates at compressed size.

The reference lets vLLM allocate its bf16 paged cache and frees it afterwards
(`free_kv_cache`, integration/vllm.py:452-501), keeping its own per-layer
Python lists of compressed chunks for ONE sequence (integration/vllm.py:139-145).
Here the cache is a first-class paged object, the way an engine wants it:

* `CompressedCacheSpec` tells the engine how many bytes a page (one 16-token
  block of all kv heads of a layer) takes - 100 bytes per token and head at
  head_dim 128 with 3-bit keys / 2-bit values instead of 512 for bf16 K+V -
  so that it sizes its block pool from free memory at COMPRESSED size;
* `CompressedPagedKVCache` is laid over the buffer the engine allocated (no
  copy, no growth), takes the engine's `slot_mapping` on writes
  (`write` = reshape_and_cache: compress-on-store of any mix of sequences in
  one launch) and the engine's `block_tables` / `seq_lens` on reads
  (`decode` = one batched launch over every sequence of the step).

Nothing here allocates per step.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import _engine as E

BLOCK_TOKENS = E.TQ_BLOCK_TOKENS


@dataclass(frozen=True)
class CompressedCacheSpec:
    """Page geometry of one layer's compressed cache (the role of vLLM's AttentionSpec)."""

    head_dim: int
    num_kv_heads: int
    key_bits: int = 3
    value_bits: int = 2
    block_size: int = BLOCK_TOKENS

    def __post_init__(self):
        if self.block_size != BLOCK_TOKENS:
            raise ValueError(f"compressed pages hold {BLOCK_TOKENS} tokens")

    @property
    def bytes_per_token(self) -> int:
        """Per kv head: codes, sign bits, two fp16 norms, value codes, fp16 group scales and zero points
        (the reference's memory_bytes accounting, store.py:116-128)."""
        return E.get_layout(self.head_dim, self.key_bits, self.value_bits).bytes_per_token

    @property
    def page_size_bytes(self) -> int:
        return self.block_size * self.num_kv_heads * self.bytes_per_token

    @property
    def bf16_page_size_bytes(self) -> int:
        """What the same page costs as bf16 K + V."""
        return self.block_size * self.num_kv_heads * self.head_dim * 2 * 2

    def num_blocks_for(self, memory_bytes: int) -> int:
        return memory_bytes // self.page_size_bytes

    def max_memory_usage_bytes(self, max_model_len: int) -> int:
        return -(-max_model_len // self.block_size) * self.page_size_bytes


class CompressedPagedKVCache:
    """One layer's compressed paged cache over engine-allocated memory."""

    def __init__(self, spec: CompressedCacheSpec, raw: torch.Tensor, layer_idx: int = 0,
                 seed: Optional[int] = None):
        self.spec = spec
        self.device = raw.device
        self.consts = E.LayerConstants(spec.head_dim, spec.key_bits, spec.value_bits, self.device,
                                       seed=42 + layer_idx * 7 if seed is None else seed)
        if self.consts.block_bytes * spec.num_kv_heads != spec.page_size_bytes:
            raise AssertionError("page size and record layout disagree")
        self.pool = E.BlockPool.over(self.consts, spec.num_kv_heads, raw)
        self.workspace = E.Workspace(self.device)

    @classmethod
    def allocate(cls, spec: CompressedCacheSpec, num_blocks: int, device, layer_idx: int = 0) -> "CompressedPagedKVCache":
        """Stand-in for the engine's allocation (tests, stand-alone use)."""
        raw = torch.zeros(num_blocks * spec.page_size_bytes, dtype=torch.uint8, device=device)
        return cls(spec, raw, layer_idx)

    @property
    def num_blocks(self) -> int:
        return self.pool.num_blocks

    def write(self, key: torch.Tensor, value: torch.Tensor, slot_mapping: torch.Tensor) -> None:
        """Compress `key` / `value` (T, H, D) into the slots the engine chose: slot = block * 16 +
        offset, negative = padding token to skip (the contract of vLLM's reshape_and_cache)."""
        t = key.shape[0]
        if slot_mapping.dtype != torch.int64 or slot_mapping.numel() < t:
            raise ValueError("slot_mapping must hold one int64 slot per token")
        if key.stride(2) != 1 or value.stride() != key.stride():
            key, value = key.contiguous(), value.contiguous()
        E.store(self.consts, self.pool, key, value, stride_token=key.stride(0), stride_head=key.stride(1), n_tokens=t,
                n_heads=self.spec.num_kv_heads, slot_mapping=slot_mapping.contiguous())

    def decode(self, query: torch.Tensor, block_tables: torch.Tensor, seq_lens: torch.Tensor, max_seq_len: int,
               scale: Optional[float] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One decode token per sequence: query (B, Qh, D), block_tables (B, max_blocks) int32, seq_lens
        (B,) int32 -> (B, Qh, D).  Every sequence of the step in one launch."""
        return E.decode(self.consts, self.pool, self.workspace, query, block_tables, seq_lens, max_seq_len,
                        scale=scale, min_history=1, out=out)


def kv_cache_specs(layer_states: dict) -> dict:
    """Spec per hooked attention layer, for an engine that sizes and allocates the cache itself
    (the alternative to allocating bf16 pages and dropping them with `free_kv_cache`)."""
    return {name: CompressedCacheSpec(st.config.head_dim, st.config.num_kv_heads, st.config.key_bits,
                                      st.config.value_bits)
            for name, st in layer_states.items() if st.supports_hybrid}

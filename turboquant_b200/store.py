"""Compressed KV store of one layer (reference store.py:19-134).

The reference keeps a Python list of quantised chunks and re-concatenates the
whole history after every append.  Here `append_chunk` compresses straight
into a pool of block records on the device (one CUDA launch, no
concatenation); the decode kernel reads the pool directly.  `get_flat_cache`
still returns the reference's flat planes for callers that want them.
"""

from __future__ import annotations

from typing import NamedTuple, Optional

import torch

from . import _engine as E
from .kv_cache import ValueQuantized
from .quantizer import ProdQuantized, TurboQuantProd


class FlatCache(NamedTuple):
    prod_q: ProdQuantized     # (num_kv_heads, total_tokens, ...)
    value_q: ValueQuantized   # (num_kv_heads, total_tokens, ...)
    num_tokens: int


class CompressedKVStore:
    def __init__(self, head_dim: int, num_kv_heads: int, key_bits: int = 3, value_bits: int = 2,
                 value_group_size: int = 32, device=None, layer_idx: int = 0, capacity_tokens: int = 4096,
                 consts: Optional[E.LayerConstants] = None):
        self.head_dim = head_dim
        self.num_kv_heads = num_kv_heads
        self.key_bits = key_bits
        self.value_bits = value_bits
        self.value_group_size = min(value_group_size, head_dim)
        self.device = torch.device(device) if device is not None else torch.device("cuda")
        self.layer_idx = layer_idx
        # `consts` lets a caller supply its own Pi / S / code book (tests feed the reference's)
        self.consts = consts if consts is not None else E.LayerConstants(
            head_dim, key_bits, value_bits, self.device, seed=42 + layer_idx * 7, group_size=self.value_group_size)
        self.quantizer = TurboQuantProd(dim=head_dim, bits=key_bits, device=self.device, seed=42 + layer_idx * 7,
                                        consts=self.consts)
        self.pool = E.BlockPool(self.consts, num_kv_heads, E.blocks_for(capacity_tokens))
        self.block_table = E.identity_block_table(self.pool.num_blocks, self.device)
        self.workspace = E.Workspace(self.device)
        self._num_tokens = 0
        self._num_chunks = 0
        self._seq_len_dev = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._seq_len_dev_val = 0          # what the device copy holds; brought up to date when it is asked for
        self._flat: Optional[FlatCache] = None

    @property
    def num_tokens(self) -> int:
        return self._num_tokens

    @property
    def num_chunks(self) -> int:
        return self._num_chunks

    @property
    def seq_len_device(self) -> torch.Tensor:
        """(1,) int32 device tensor holding num_tokens (what the decode kernel reads).  The device copy is
        refreshed HERE, not by every append (a fill between two store launches would keep the second from
        starting under the first): ask for it after the last append, on the stream the decode will use."""
        if self._seq_len_dev_val != self._num_tokens:
            self._seq_len_dev.fill_(self._num_tokens)
            self._seq_len_dev_val = self._num_tokens
        return self._seq_len_dev

    def reserve(self, n_tokens: int) -> None:
        """Make room for `n_tokens` in total (doubling growth)."""
        need = E.blocks_for(n_tokens)
        if need > self.pool.num_blocks:
            self.pool.resize(max(need, 2 * self.pool.num_blocks))
            self.block_table = E.identity_block_table(self.pool.num_blocks, self.device)

    def append_chunk(self, key: torch.Tensor, value: torch.Tensor) -> None:
        """Compress and append key/value of shape (chunk_len, num_kv_heads, head_dim)."""
        t = key.shape[0]
        if t == 0:
            return
        if key.shape != value.shape or key.shape[1] != self.num_kv_heads or key.shape[2] != self.head_dim:
            raise ValueError(f"expected (T, {self.num_kv_heads}, {self.head_dim}) key and value, got "
                             f"{tuple(key.shape)} / {tuple(value.shape)}")
        if key.stride(2) != 1 or value.stride() != key.stride():
            key, value = key.contiguous(), value.contiguous()
        self.reserve(self._num_tokens + t)
        E.store(self.consts, self.pool, key, value, stride_token=key.stride(0), stride_head=key.stride(1),
                n_tokens=t, n_heads=self.num_kv_heads, block_table=self.block_table, start_pos=self._num_tokens)
        self._num_tokens += t
        self._num_chunks += 1
        self._flat = None

    def append_from_paged(self, key_cache: torch.Tensor, value_cache: torch.Tensor, src_block_table: torch.Tensor,
                          num_tokens: int) -> None:
        """Compress and append the first `num_tokens` tokens of a sequence held in a paged cache
        ((num_blocks, block_size, H, D) planes, `src_block_table` logical -> physical block): what
        `append_chunk` does to the gathered rows, without gathering them when the table-walking kernel
        takes the call.  No reference counterpart as a single call (capture.py:187-217 gathers first)."""
        if num_tokens == 0:
            return
        if key_cache.shape[2] != self.num_kv_heads or key_cache.shape[3] != self.head_dim:
            raise ValueError(f"expected (num_blocks, block_size, {self.num_kv_heads}, {self.head_dim}) planes")
        self.reserve(self._num_tokens + num_tokens)
        table = src_block_table.to(device=self.device, dtype=torch.int32).contiguous()
        if not E.store_paged(self.consts, self.pool, key_cache, value_cache, src_block_table=table,
                             n_tokens=num_tokens, block_table=self.block_table, start_pos=self._num_tokens):
            bs = key_cache.shape[1]
            phys = table[:(num_tokens + bs - 1) // bs].long()
            k = key_cache.index_select(0, phys).flatten(0, 1)[:num_tokens]
            v = value_cache.index_select(0, phys).flatten(0, 1)[:num_tokens]
            return self.append_chunk(k, v)
        self._num_tokens += num_tokens
        self._num_chunks += 1
        self._flat = None

    def get_flat_cache(self) -> Optional[FlatCache]:
        """The reference's flat planes (H, N, ...), rebuilt after a write."""
        if self._num_tokens == 0:
            return None
        if self._flat is None:
            ps = E.pool_to_planes(self.consts, self.pool, self.block_table, self._num_tokens)
            self._flat = FlatCache(
                ProdQuantized(ps.mse_indices, ps.qjl_signs, ps.residual_norms, ps.norms, self.key_bits - 1),
                ValueQuantized(ps.v_data, ps.v_scales, ps.v_zeros, self.value_bits),
                self._num_tokens)
        return self._flat

    def memory_bytes(self) -> int:
        """Codes plus two bytes per norm / scale / zero point (reference store.py:116-128)."""
        return self._num_tokens * self.num_kv_heads * self.consts.bytes_per_token

    def reset(self) -> None:
        self._num_tokens = 0
        self._num_chunks = 0
        self._seq_len_dev.zero_()
        self._seq_len_dev_val = 0
        self._flat = None

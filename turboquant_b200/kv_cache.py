"""Value group quantisation and the legacy single-object KV cache
(reference kv_cache.py:20-349), computed by the CUDA library.
"""

from __future__ import annotations

import math
from typing import NamedTuple, Optional

import torch

from . import _engine as E


class ValueQuantized(NamedTuple):
    data: torch.Tensor     # (..., n_tokens, packed_d) uint8
    scales: torch.Tensor   # (..., n_tokens, n_groups)
    zeros: torch.Tensor    # (..., n_tokens, n_groups)
    bits: int = 2


_CONSTS: dict[tuple, E.LayerConstants] = {}


def _value_consts(d: int, bits: int, device) -> E.LayerConstants:
    key = (d, bits, str(device))
    if key not in _CONSTS:
        _CONSTS[key] = E.LayerConstants(d, 3, bits, device)
    return _CONSTS[key]


def unpack_values(vq: ValueQuantized) -> torch.Tensor:
    """One uint8 per element from the packed bytes (pure bit slicing)."""
    bits = vq.bits if len(vq) > 3 else 2
    p = vq.data
    if bits == 2:
        parts = [(p >> s) & 0x03 for s in (0, 2, 4, 6)]
    elif bits == 4:
        parts = [(p >> s) & 0x0F for s in (0, 4)]
    else:
        return p
    return torch.stack(parts, dim=-1).reshape(*p.shape[:-1], p.shape[-1] * len(parts))


def quantize_values(v: torch.Tensor, bits: int = 2, group_size: int = 32) -> ValueQuantized:
    """Per-group (32) asymmetric min/max quantisation of (..., seq, d) values.

    Scales and zero points are returned in v's dtype after their fp16 round
    trip through the compressed record.
    """
    if group_size != 32:
        raise ValueError("only value groups of 32 are compiled")
    E.require_cuda(v, "v")
    d = v.shape[-1]
    consts = _value_consts(d, bits, v.device)
    lead = v.shape[:-1]
    v2 = v.reshape(-1, d)
    if v2.stride(-1) != 1:
        v2 = v2.contiguous()
    n = v2.shape[0]
    pool = E.BlockPool(consts, 1, E.blocks_for(n))
    bt = E.identity_block_table(pool.num_blocks, v.device)
    E.store(consts, pool, v2, v2, stride_token=v2.stride(0), stride_head=0, n_tokens=n, n_heads=1,
            block_table=bt, start_pos=0)
    ps = E.pool_to_planes(consts, pool, bt, n)
    return ValueQuantized(ps.v_data[0].reshape(*lead, -1), ps.v_scales[0].reshape(*lead, -1).to(v.dtype),
                          ps.v_zeros[0].reshape(*lead, -1).to(v.dtype), bits)


def dequantize_values(vq: ValueQuantized, group_size: int = 32) -> torch.Tensor:
    """code * scale + zero in fp32, (..., seq, d)."""
    bits = vq.bits if len(vq) > 3 else 2
    data = vq.data
    E.require_cuda(data, "vq.data")
    d = data.shape[-1] * (4 if bits == 2 else 2)
    consts = _value_consts(d, bits, data.device)
    lay = consts.layout
    n = data.shape[-2]
    heads = max(1, data.numel() // (n * data.shape[-1]))
    dev = data.device
    ps = E.PlaneSet.from_tensors(
        consts, torch.zeros(heads, n, lay.kcode_row, dtype=torch.uint8, device=dev),
        torch.zeros(heads, n, lay.ksign_row, dtype=torch.uint8, device=dev),
        torch.zeros(heads, n, device=dev), torch.zeros(heads, n, device=dev),
        data.reshape(heads, n, -1), vq.scales.reshape(heads, n, -1), vq.zeros.reshape(heads, n, -1))
    pool = E.BlockPool(consts, heads, E.blocks_for(n))
    bt = E.identity_block_table(pool.num_blocks, dev)
    E.planes_to_pool(consts, ps, n, pool, bt)
    return E.dequant_values(consts, pool, bt, n).reshape(*data.shape[:-1], d)


class TurboQuantKVCache:
    """Legacy cache object: quantised history plus an exact buffer of the last
    `buffer_size` tokens, for tensors of shape (batch, heads, seq, head_dim).

    prefill / append / attention_scores / attend / memory_bytes /
    get_seq_length behave as in the reference (kv_cache.py:119-349); the oldest
    buffered token is compressed whenever the buffer overflows.
    """

    def __init__(self, head_dim: int, key_bits: int = 3, value_bits: int = 2, value_group_size: int = 32,
                 buffer_size: int = 128, device=None, dtype: torch.dtype = torch.float16, layer_idx: int = 0):
        from .quantizer import TurboQuantProd
        self.head_dim, self.key_bits, self.value_bits = head_dim, key_bits, value_bits
        self.value_group_size, self.buffer_size = value_group_size, buffer_size
        self.device = torch.device(device) if device is not None else torch.device("cuda")
        self.dtype, self.layer_idx = dtype, layer_idx
        self.consts = E.LayerConstants(head_dim, key_bits, value_bits, self.device, seed=42 + layer_idx * 7)
        self.key_quantizer = TurboQuantProd(head_dim, key_bits, self.device, seed=42 + layer_idx * 7,
                                            consts=self.consts)
        self.seq_len = 0
        self.key_buffer: Optional[torch.Tensor] = None
        self.value_buffer: Optional[torch.Tensor] = None
        self._pool: Optional[E.BlockPool] = None
        self._bt: Optional[torch.Tensor] = None
        self._n_quant = 0
        self._lead: Optional[tuple] = None   # (batch, heads)
        self._ws = E.Workspace(self.device)

    # -- compressed segment ---------------------------------------------------
    def _append_compressed(self, keys: torch.Tensor, values: torch.Tensor) -> None:
        b, h, t, d = keys.shape
        if self._pool is None:
            self._lead = (b, h)
            self._pool = E.BlockPool(self.consts, b * h, E.blocks_for(max(t, 1024)))
            self._bt = E.identity_block_table(self._pool.num_blocks, self.device)
        need = E.blocks_for(self._n_quant + t)
        if need > self._pool.num_blocks:
            self._pool.resize(max(need, 2 * self._pool.num_blocks))
            self._bt = E.identity_block_table(self._pool.num_blocks, self.device)
        k = keys.contiguous()
        v = values.contiguous()
        # (b, h, t, d) contiguous: head index b*h+h' has stride t*d, tokens stride d
        E.store(self.consts, self._pool, k, v, stride_token=d, stride_head=t * d, n_tokens=t, n_heads=b * h,
                block_table=self._bt, start_pos=self._n_quant)
        self._n_quant += t

    @property
    def key_quantized(self):
        if self._n_quant == 0:
            return None
        from .quantizer import ProdQuantized
        ps = E.pool_to_planes(self.consts, self._pool, self._bt, self._n_quant)
        b, h = self._lead
        return ProdQuantized(ps.mse_indices.reshape(b, h, self._n_quant, -1),
                             ps.qjl_signs.reshape(b, h, self._n_quant, -1),
                             ps.residual_norms.reshape(b, h, -1).float(), ps.norms.reshape(b, h, -1),
                             self.key_bits - 1)

    @property
    def value_quantized(self):
        if self._n_quant == 0:
            return None
        ps = E.pool_to_planes(self.consts, self._pool, self._bt, self._n_quant)
        b, h = self._lead
        return ValueQuantized(ps.v_data.reshape(b, h, self._n_quant, -1), ps.v_scales.reshape(b, h, self._n_quant, -1),
                              ps.v_zeros.reshape(b, h, self._n_quant, -1), self.value_bits)

    # -- reference API ---------------------------------------------------------
    def prefill(self, keys: torch.Tensor, values: torch.Tensor) -> None:
        seq_len = keys.shape[-2]
        self.seq_len = seq_len
        if seq_len <= self.buffer_size:
            self.key_buffer, self.value_buffer = keys, values
            return
        n_quant = seq_len - self.buffer_size
        self.key_buffer, self.value_buffer = keys[..., n_quant:, :], values[..., n_quant:, :]
        self._append_compressed(keys[..., :n_quant, :], values[..., :n_quant, :])

    def append(self, key: torch.Tensor, value: torch.Tensor) -> None:
        self.seq_len += 1
        if self.key_buffer is not None:
            self.key_buffer = torch.cat([self.key_buffer, key], dim=-2)
            self.value_buffer = torch.cat([self.value_buffer, value], dim=-2)
        else:
            self.key_buffer, self.value_buffer = key, value
        n_flush = self.key_buffer.shape[-2] - self.buffer_size
        if n_flush > 0:
            self._append_compressed(self.key_buffer[..., :n_flush, :], self.value_buffer[..., :n_flush, :])
            self.key_buffer = self.key_buffer[..., n_flush:, :]
            self.value_buffer = self.value_buffer[..., n_flush:, :]

    def attention_scores(self, query: torch.Tensor, scale: float = None) -> torch.Tensor:
        """query (batch, heads, n_q, d) -> logits (batch, heads, n_q, seq_len)."""
        if scale is None:
            scale = 1.0 / math.sqrt(self.head_dim)
        parts = []
        if self._n_quant > 0:
            b, h = self._lead
            q3 = query.reshape(b * h, query.shape[-2], self.head_dim)
            logits = E.scores(self.consts, self._pool, self._ws, self._bt, self._n_quant, q3)
            parts.append(logits.reshape(b, h, query.shape[-2], self._n_quant) * scale)
        if self.key_buffer is not None:
            parts.append(torch.matmul(query, self.key_buffer.transpose(-2, -1)) * scale)
        return torch.cat([p.to(parts[0].dtype) for p in parts], dim=-1)

    def attend(self, attn_weights: torch.Tensor) -> torch.Tensor:
        """softmaxed weights (batch, heads, n_q, seq_len) -> (batch, heads, n_q, d)."""
        outs, col = [], 0
        if self._n_quant > 0:
            b, h = self._lead
            v = E.dequant_values(self.consts, self._pool, self._bt, self._n_quant).reshape(b, h, self._n_quant, -1)
            w = attn_weights[..., col: col + self._n_quant]
            outs.append(torch.matmul(w.float(), v))
            col += self._n_quant
        if self.value_buffer is not None:
            n_buf = self.value_buffer.shape[-2]
            w = attn_weights[..., col: col + n_buf]
            outs.append(torch.matmul(w.to(self.value_buffer.dtype), self.value_buffer).to(outs[0].dtype if outs else w.dtype))
        return sum(outs)

    def memory_bytes(self) -> dict:
        info = {"quantized_keys": 0, "quantized_values": 0, "buffer": 0, "total": 0}
        if self._n_quant > 0:
            lay = self.consts.layout
            rows = self._n_quant * self._lead[0] * self._lead[1]
            info["quantized_keys"] = rows * (lay.kcode_row + lay.ksign_row + 4)
            info["quantized_values"] = rows * (lay.vcode_row + 4 * lay.n_groups)
        if self.key_buffer is not None:
            info["buffer"] += self.key_buffer.nelement() * 2
        if self.value_buffer is not None:
            info["buffer"] += self.value_buffer.nelement() * 2
        info["total"] = info["quantized_keys"] + info["quantized_values"] + info["buffer"]
        return info

    def get_seq_length(self) -> int:
        return self.seq_len

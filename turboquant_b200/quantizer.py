"""TurboQuant quantisers with the reference's names and result types
(reference quantizer.py:22-35,93-306), computed by the CUDA library.

Differences a caller can observe: norms and residual norms come back rounded
to fp16 (the storage format of the compressed record) and cast to the input
dtype, and only the compiled shapes are accepted (head_dim 128/256, MSE codes
of 2 or 3 bits).
"""

from __future__ import annotations

from typing import NamedTuple, Optional

import torch

from . import _engine as E


class MSEQuantized(NamedTuple):
    indices: torch.Tensor   # (..., packed_len) uint8
    norms: torch.Tensor     # (...,)
    bits: int


class ProdQuantized(NamedTuple):
    mse_indices: torch.Tensor     # (..., packed_len) uint8
    qjl_signs: torch.Tensor       # (..., d/8) uint8
    residual_norms: torch.Tensor  # (...,)
    norms: torch.Tensor           # (...,)
    mse_bits: int


def _rows(x: torch.Tensor):
    """View (..., d) as (rows, d) for a one-head store."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    return lead, x2


class _QuantizerBase(torch.nn.Module):
    def __init__(self, dim: int, key_bits: int, device, seed: int, consts: Optional[E.LayerConstants] = None):
        super().__init__()
        self.dim = dim
        self.device = torch.device(device) if device is not None else torch.device("cuda")
        self.seed = seed
        self.consts = consts if consts is not None else E.LayerConstants(dim, key_bits, 2, self.device, seed=seed)
        self._ws = E.Workspace(self.device)
        # buffers with the reference's attribute names
        self.register_buffer("Pi", self.consts.Pi, persistent=False)
        self.register_buffer("centroids", self.consts.centroids, persistent=False)
        self.register_buffer("boundaries", self.consts.boundaries, persistent=False)
        self.register_buffer("decision_boundaries", self.consts.boundaries[1:-1].contiguous(), persistent=False)

    def _compress_rows(self, x2: torch.Tensor):
        """Store (rows, d) as one head; returns (pool, block table, planes)."""
        n = x2.shape[0]
        pool = E.BlockPool(self.consts, 1, E.blocks_for(n))
        bt = E.identity_block_table(pool.num_blocks, self.device)
        # the value half of the record is not used here: feed the keys as values
        E.store(self.consts, pool, x2, x2, stride_token=x2.stride(0), stride_head=0, n_tokens=n, n_heads=1,
                block_table=bt, start_pos=0)
        return pool, bt, E.pool_to_planes(self.consts, pool, bt, n)

    def _pool_from(self, mse_indices, qjl_signs, norms, residual_norms):
        """Scatter packed keys (..., n, packed) into a (heads = prod(...), n) pool."""
        lay = self.consts.layout
        n = mse_indices.shape[-2]
        heads = max(1, mse_indices.numel() // (n * mse_indices.shape[-1]))
        dev = self.device
        zeros_v = torch.zeros(heads, n, lay.vcode_row, dtype=torch.uint8, device=dev)
        zeros_g = torch.zeros(heads, n, lay.n_groups, dtype=torch.float16, device=dev)
        if qjl_signs is None:
            qjl_signs = torch.zeros(heads, n, lay.ksign_row, dtype=torch.uint8, device=dev)
            residual_norms = torch.zeros(heads, n, device=dev)
        ps = E.PlaneSet.from_tensors(self.consts, mse_indices.reshape(heads, n, -1), qjl_signs.reshape(heads, n, -1),
                                     norms.reshape(heads, n), residual_norms.reshape(heads, n), zeros_v, zeros_g,
                                     zeros_g)
        pool = E.BlockPool(self.consts, heads, E.blocks_for(n))
        bt = E.identity_block_table(pool.num_blocks, dev)
        E.planes_to_pool(self.consts, ps, n, pool, bt)
        return pool, bt, heads, n


class TurboQuantMSE(_QuantizerBase):
    """Algorithm 1: normalise, rotate, nearest centroid per coordinate."""

    def __init__(self, dim: int, bits: int = 3, device=None, dtype: torch.dtype = torch.float32, seed: int = 42,
                 consts: Optional[E.LayerConstants] = None):
        super().__init__(dim, bits + 1, device, seed, consts)
        self.bits = bits
        self.n_clusters = 2 ** bits

    def quantize(self, x: torch.Tensor) -> MSEQuantized:
        lead, x2 = _rows(x)
        _, _, ps = self._compress_rows(x2)
        return MSEQuantized(ps.mse_indices[0].reshape(*lead, -1), ps.norms[0].reshape(lead).to(x.dtype), self.bits)

    def dequantize(self, q: MSEQuantized) -> torch.Tensor:
        pool, bt, heads, n = self._pool_from(q.indices, None, q.norms, None)
        out = E.dequant_keys(self.consts, pool, bt, n, with_qjl=False)
        return out.reshape(*q.norms.shape, self.dim)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.dequantize(self.quantize(x))


class TurboQuantProd(_QuantizerBase):
    """Algorithm 2: MSE stage at bits-1, then a 1-bit QJL sketch of the residual."""

    def __init__(self, dim: int, bits: int = 3, device=None, dtype: torch.dtype = torch.float32, seed: int = 42,
                 consts: Optional[E.LayerConstants] = None):
        assert bits >= 2, "Inner product TurboQuant requires at least 2 bits (1 for MSE + 1 for QJL)"
        super().__init__(dim, bits, device, seed, consts)
        self.bits = bits
        self.qjl_scale = self.consts.qjl_scale
        self.register_buffer("S", self.consts.S, persistent=False)
        self._mse: Optional[TurboQuantMSE] = None

    @property
    def mse_quantizer(self) -> TurboQuantMSE:
        """The stage-1 quantiser (bits-1), sharing this object's constants."""
        if self._mse is None:
            object.__setattr__(self, "_mse", TurboQuantMSE(self.dim, self.bits - 1, self.device, seed=self.seed,
                                                           consts=self.consts))
        return self._mse

    def quantize(self, x: torch.Tensor) -> ProdQuantized:
        lead, x2 = _rows(x)
        _, _, ps = self._compress_rows(x2)
        return ProdQuantized(ps.mse_indices[0].reshape(*lead, -1), ps.qjl_signs[0].reshape(*lead, -1),
                             ps.residual_norms[0].reshape(lead).float(), ps.norms[0].reshape(lead).to(x.dtype),
                             self.bits - 1)

    def dequantize(self, q: ProdQuantized) -> torch.Tensor:
        pool, bt, heads, n = self._pool_from(q.mse_indices, q.qjl_signs, q.norms, q.residual_norms)
        out = E.dequant_keys(self.consts, pool, bt, n, with_qjl=True)
        return out.reshape(*q.norms.shape, self.dim)

    def attention_score(self, query: torch.Tensor, quantized_key: ProdQuantized) -> torch.Tensor:
        """query (..., n_q, d), keys (..., n_k, ...) -> unscaled logits (..., n_q, n_k)."""
        pool, bt, heads, n = self._pool_from(quantized_key.mse_indices, quantized_key.qjl_signs,
                                             quantized_key.norms, quantized_key.residual_norms)
        n_q = query.shape[-2]
        q3 = query.reshape(-1, n_q, self.dim)
        if q3.shape[0] != heads:
            q3 = q3.expand(heads, n_q, self.dim)
        logits = E.scores(self.consts, pool, self._ws, bt, n, q3.contiguous())
        return logits.reshape(*quantized_key.norms.shape[:-1], n_q, n)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.dequantize(self.quantize(x))

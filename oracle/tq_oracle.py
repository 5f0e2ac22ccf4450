"""CPU oracle for the TurboQuant KV-cache hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, with torch CPU ops and numpy, the arithmetic of the
reference implementation (0xSero/turboquant) for the compress-on-store
pipeline and the decode attention over compressed K/V.  It is the checker
for the CUDA path; nothing in the product package imports it.  Only the
test-suite, the smoke entry and the benchmark's CPU-baseline legs may
import this file.

Why torch CPU ops: the reference's arithmetic *is* torch (matmul, norm,
searchsorted, round, softmax) - a third-party dependency of the reference
(setup.py:15 `torch>=2.1`, no pin; this image has 2.11.0).  Using the same
library calls on the same CPU makes the oracle reproduce the reference to
the bit; the integer stages (bucket search, bit packing) are restated in
numpy.

Parity pin: the reference ships no tests, fixtures or golden vectors.  The
oracle is therefore pinned against outputs of the reference itself, executed
in the build container, stored under tests/golden/ together with the script
that produced them (tests/golden/make_golden.py), and against the code-book
constants the reference ships as JSON data.

Each function cites the reference file:line it follows.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

MIN_HISTORY_FOR_TQ = 16  # score.py:26


# --------------------------------------------------------------------------
# constants (rotation.py, codebook.py)
# --------------------------------------------------------------------------

def rotation_matrix(d: int, seed: int) -> torch.Tensor:
    """Pi = Q * sign(diag R) of QR(randn(d,d)) on a seeded CPU generator.

    rotation.py:17-40.  LAPACK's QR may differ in the last bits between CPU
    models, which is why the golden fixtures carry Pi itself.
    """
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    gauss = torch.randn(d, d, generator=g, dtype=torch.float32)
    q, r = torch.linalg.qr(gauss)
    return (q * torch.sign(torch.diag(r)).unsqueeze(0)).contiguous()


def qjl_matrix(d: int, seed: int) -> torch.Tensor:
    """S = randn(d,d) on a seeded CPU generator.  rotation.py:43-56."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return torch.randn(d, d, generator=g, dtype=torch.float32)


def layer_seeds(layer_idx: int) -> tuple[int, int]:
    """(Pi seed, S seed) of a layer.  store.py:56, quantizer.py:208."""
    base = 42 + 7 * layer_idx
    return base, base + 1000


def qjl_scale(d: int) -> float:
    """sqrt(pi/2)/d.  quantizer.py:212."""
    return math.sqrt(math.pi / 2.0) / d


# --------------------------------------------------------------------------
# integer stages: bucket search and bit packing (numpy)
# --------------------------------------------------------------------------

def bucket_indices(y: np.ndarray, interior_boundaries: np.ndarray) -> np.ndarray:
    """idx = #{i : b_i < y}  (searchsorted, side='left').  quantizer.py:144."""
    return np.searchsorted(interior_boundaries.astype(np.float32),
                           y.astype(np.float32), side="left").astype(np.uint8)


def _pack_params(bits: int) -> tuple[int, int]:
    """(field width, values per byte).  quantizer.py:50-59."""
    if bits == 1:
        return 1, 8
    if bits == 2:
        return 2, 4
    if bits <= 4:
        return 4, 2
    raise ValueError("bits > 4 are stored unpacked by the reference")


def pack_indices(idx: np.ndarray, bits: int) -> np.ndarray:
    """LSB-first packing; 3-bit codes occupy nibbles.  quantizer.py:38-69."""
    width, vpb = _pack_params(bits)
    d = idx.shape[-1]
    pad = (-d) % vpb
    a = idx.astype(np.uint8)
    if pad:
        a = np.concatenate([a, np.zeros(a.shape[:-1] + (pad,), np.uint8)], -1)
    a = a.reshape(a.shape[:-1] + (-1, vpb)).astype(np.uint32)
    shifts = (np.arange(vpb, dtype=np.uint32) * width)
    return ((a << shifts).sum(-1) & 0xFF).astype(np.uint8)


def unpack_indices(packed: np.ndarray, bits: int, d: int) -> np.ndarray:
    """Inverse of pack_indices.  quantizer.py:72-90."""
    width, vpb = _pack_params(bits)
    shifts = (np.arange(vpb, dtype=np.uint8) * width).astype(np.uint8)
    out = (packed[..., None] >> shifts) & ((1 << width) - 1)
    return out.reshape(packed.shape[:-1] + (-1,))[..., :d].astype(np.uint8)


def pack_signs(projected: np.ndarray) -> np.ndarray:
    """bit j of byte i = (p[8i+j] > 0).  quantizer.py:214-222."""
    bits = (projected > 0).astype(np.uint8)
    d = bits.shape[-1]
    pad = (-d) % 8
    if pad:
        bits = np.concatenate([bits, np.zeros(bits.shape[:-1] + (pad,), np.uint8)], -1)
    return np.packbits(bits, axis=-1, bitorder="little")


def unpack_signs(packed: np.ndarray, d: int) -> np.ndarray:
    """+1.0 / -1.0 per coordinate.  quantizer.py:224-229."""
    bits = np.unpackbits(packed, axis=-1, bitorder="little")[..., :d]
    return (2.0 * bits.astype(np.float32) - 1.0).astype(np.float32)


def pack_values(vq: np.ndarray, bits: int) -> np.ndarray:
    """2-bit: a|b<<2|c<<4|d<<6; 4-bit: a|b<<4.  kv_cache.py:80-90."""
    if bits == 2:
        v = vq.reshape(vq.shape[:-1] + (-1, 4))
        return (v[..., 0] | (v[..., 1] << 2) | (v[..., 2] << 4) | (v[..., 3] << 6)).astype(np.uint8)
    if bits == 4:
        v = vq.reshape(vq.shape[:-1] + (-1, 2))
        return (v[..., 0] | (v[..., 1] << 4)).astype(np.uint8)
    raise ValueError("value bits must be 2 or 4")


def unpack_values(data: np.ndarray, bits: int) -> np.ndarray:
    """kv_cache.py:28-42."""
    if bits == 2:
        parts = [(data >> s) & 3 for s in (0, 2, 4, 6)]
    elif bits == 4:
        parts = [(data >> s) & 15 for s in (0, 4)]
    else:
        raise ValueError("value bits must be 2 or 4")
    return np.stack(parts, -1).reshape(data.shape[:-1] + (-1,)).astype(np.uint8)


# --------------------------------------------------------------------------
# key path (quantizer.py)
# --------------------------------------------------------------------------

@dataclass
class KeyStages:
    """Every intermediate of TurboQuantProd.quantize, for stage-level parity."""
    norms: torch.Tensor        # (...,) in x's dtype
    x_unit: torch.Tensor       # (..., d) in x's dtype
    y: torch.Tensor            # (..., d) fp32 rotated unit vector
    idx: np.ndarray            # (..., d) uint8
    packed: np.ndarray         # (..., d*w/8) uint8
    x_hat: torch.Tensor        # (..., d) fp32 MSE reconstruction
    residual_norms: torch.Tensor  # (...,) fp32
    projected: torch.Tensor    # (..., d) fp32
    signs: np.ndarray          # (..., d/8) uint8


def mse_quantize(x: torch.Tensor, pi: torch.Tensor, boundaries: torch.Tensor, bits: int):
    """TurboQuantMSE.quantize, quantizer.py:129-149.

    `boundaries` holds the 2^bits+1 edges; the interior ones decide.
    Norm and normalisation run in x's dtype (bf16 stays bf16), the rotation
    in fp32.
    """
    norms = x.norm(dim=-1, keepdim=False)
    x_unit = x / (norms.unsqueeze(-1) + 1e-10)
    y = torch.matmul(x_unit.float(), pi.T)
    interior = boundaries[1:-1].to(torch.float32).numpy()
    idx = bucket_indices(y.contiguous().numpy(), interior)
    return norms, x_unit, y, idx, pack_indices(idx, bits)


def mse_dequantize(idx: np.ndarray, norms: torch.Tensor, pi: torch.Tensor,
                   centroids: torch.Tensor) -> torch.Tensor:
    """centroids[idx] @ Pi * norms.  quantizer.py:151-165."""
    y_hat = centroids.to(torch.float32)[torch.from_numpy(idx.astype(np.int64))]
    return torch.matmul(y_hat, pi) * norms.unsqueeze(-1)


def prod_quantize(x: torch.Tensor, pi: torch.Tensor, s: torch.Tensor,
                  centroids: torch.Tensor, boundaries: torch.Tensor,
                  key_bits: int) -> KeyStages:
    """TurboQuantProd.quantize, quantizer.py:231-257 (MSE stage at key_bits-1)."""
    mse_bits = key_bits - 1
    norms, x_unit, y, idx, packed = mse_quantize(x, pi, boundaries, mse_bits)
    x_hat = mse_dequantize(idx, norms, pi, centroids)
    residual = x - x_hat
    rnorm = residual.norm(dim=-1)
    projected = torch.matmul(residual.float(), s.T)
    signs = pack_signs(projected.numpy())
    return KeyStages(norms, x_unit, y, idx, packed, x_hat, rnorm, projected, signs)


def prod_dequantize(packed: np.ndarray, signs: np.ndarray, norms: torch.Tensor,
                    rnorms: torch.Tensor, pi: torch.Tensor, s: torch.Tensor,
                    centroids: torch.Tensor, mse_bits: int) -> torch.Tensor:
    """TurboQuantProd.dequantize, quantizer.py:259-272."""
    d = pi.shape[0]
    idx = unpack_indices(packed, mse_bits, d)
    x_mse = mse_dequantize(idx, norms, pi, centroids)
    sg = torch.from_numpy(unpack_signs(signs, d))
    x_qjl = torch.matmul(sg, s) * (qjl_scale(d) * rnorms.unsqueeze(-1))
    return x_mse + x_qjl


def attention_score(query: torch.Tensor, packed: np.ndarray, signs: np.ndarray,
                    norms: torch.Tensor, rnorms: torch.Tensor, pi: torch.Tensor,
                    s: torch.Tensor, centroids: torch.Tensor, mse_bits: int) -> torch.Tensor:
    """TurboQuantProd.attention_score (unscaled logits), quantizer.py:274-302."""
    d = pi.shape[0]
    idx = unpack_indices(packed, mse_bits, d)
    k_mse = mse_dequantize(idx, norms, pi, centroids)
    scores_mse = torch.matmul(query.float(), k_mse.float().transpose(-2, -1))
    q_sk = torch.matmul(query.float(), s.T)
    sg = torch.from_numpy(unpack_signs(signs, d))
    scores_qjl = torch.matmul(q_sk, sg.transpose(-2, -1))
    scores_qjl = scores_qjl * (qjl_scale(d) * rnorms.unsqueeze(-2))
    return scores_mse + scores_qjl.to(scores_mse.dtype)


# --------------------------------------------------------------------------
# value path (kv_cache.py)
# --------------------------------------------------------------------------

def quantize_values(v: torch.Tensor, bits: int = 2, group_size: int = 32):
    """Per-group asymmetric min/max quantisation in v's dtype, kv_cache.py:45-98.

    Returns (data uint8 ndarray, scales, zeros) with scales/zeros in v's dtype.
    """
    shape = v.shape
    d = shape[-1]
    n_groups = d // group_size
    vg = v.reshape(*shape[:-1], n_groups, group_size)
    v_min = vg.min(dim=-1, keepdim=True).values
    v_max = vg.max(dim=-1, keepdim=True).values
    n_levels = 2 ** bits - 1
    scale = ((v_max - v_min) / n_levels).clamp(min=1e-10)
    zero = v_min
    vq = ((vg - zero) / scale).round().clamp(0, n_levels).to(torch.uint8)
    data = pack_values(vq.reshape(*shape[:-1], d).numpy(), bits)
    return data, scale.squeeze(-1), zero.squeeze(-1)


def dequantize_values(data: np.ndarray, scales: torch.Tensor, zeros: torch.Tensor,
                      bits: int, group_size: int = 32) -> torch.Tensor:
    """q*scale+zero in fp32.  kv_cache.py:101-116."""
    q = torch.from_numpy(unpack_values(data, bits)).float()
    d = q.shape[-1]
    qg = q.reshape(*q.shape[:-1], d // group_size, group_size)
    out = qg * scales.unsqueeze(-1) + zeros.unsqueeze(-1)
    return out.reshape(*q.shape[:-1], d)


# --------------------------------------------------------------------------
# store (store.py) and read path (score.py)
# --------------------------------------------------------------------------

@dataclass
class Planes:
    """Flat compressed planes of one layer, (H, N, ...) like store.py:19-23."""
    mse_indices: np.ndarray      # (H, N, D*w/8) uint8
    qjl_signs: np.ndarray        # (H, N, D/8) uint8
    norms: torch.Tensor          # (H, N) x dtype
    residual_norms: torch.Tensor  # (H, N) fp32
    v_data: np.ndarray           # (H, N, D*vb/8) uint8
    v_scales: torch.Tensor       # (H, N, D/32) v dtype
    v_zeros: torch.Tensor        # (H, N, D/32) v dtype
    mse_bits: int
    v_bits: int

    @property
    def num_tokens(self) -> int:
        return int(self.mse_indices.shape[1])

    def memory_bytes(self) -> int:
        """Codes + 2 bytes per norm/scale/zero.  store.py:116-128."""
        return int(self.mse_indices.size + self.qjl_signs.size
                   + 2 * (self.norms.numel() + self.residual_norms.numel())
                   + self.v_data.size + 2 * (self.v_scales.numel() + self.v_zeros.numel()))


class OracleStore:
    """CompressedKVStore restated: append_chunk / get_flat_cache.  store.py:26-134."""

    def __init__(self, head_dim: int, num_kv_heads: int, key_bits: int, value_bits: int,
                 centroids: torch.Tensor, boundaries: torch.Tensor,
                 pi: Optional[torch.Tensor] = None, s: Optional[torch.Tensor] = None,
                 layer_idx: int = 0, value_group_size: int = 32):
        self.head_dim = head_dim
        self.num_kv_heads = num_kv_heads
        self.key_bits = key_bits
        self.value_bits = value_bits
        self.value_group_size = min(value_group_size, head_dim)
        seed_pi, seed_s = layer_seeds(layer_idx)
        self.pi = pi if pi is not None else rotation_matrix(head_dim, seed_pi)
        self.s = s if s is not None else qjl_matrix(head_dim, seed_s)
        self.centroids = centroids
        self.boundaries = boundaries
        self._chunks: list[Planes] = []

    @property
    def num_tokens(self) -> int:
        return sum(c.num_tokens for c in self._chunks)

    def append_chunk(self, key: torch.Tensor, value: torch.Tensor) -> KeyStages:
        """key/value (T, H, D) -> one chunk of planes.  store.py:73-90."""
        k = key.transpose(0, 1)   # (H, T, D); the reference's leading 1 is dropped again on flatten
        v = value.transpose(0, 1)
        st = prod_quantize(k, self.pi, self.s, self.centroids, self.boundaries, self.key_bits)
        data, scales, zeros = quantize_values(v, self.value_bits, self.value_group_size)
        self._chunks.append(Planes(st.packed, st.signs, st.norms, st.residual_norms,
                                   data, scales, zeros, self.key_bits - 1, self.value_bits))
        return st

    def get_flat_cache(self) -> Optional[Planes]:
        """Concatenate chunks along the token axis.  store.py:92-114,159-178."""
        if not self._chunks:
            return None
        c = self._chunks
        if len(c) == 1:
            return c[0]
        flat = Planes(
            np.concatenate([x.mse_indices for x in c], 1),
            np.concatenate([x.qjl_signs for x in c], 1),
            torch.cat([x.norms for x in c], 1),
            torch.cat([x.residual_norms for x in c], 1),
            np.concatenate([x.v_data for x in c], 1),
            torch.cat([x.v_scales for x in c], 1),
            torch.cat([x.v_zeros for x in c], 1),
            c[0].mse_bits, c[0].v_bits)
        self._chunks = [flat]
        return flat


def matmul_attend(query: torch.Tensor, keys: torch.Tensor, values: torch.Tensor,
                  num_kv_heads: int, scale: float) -> torch.Tensor:
    """GQA softmax attention in fp32, cast to the query dtype.  score.py:138-173.

    query (T, Qh, D); keys/values (H, N, D).
    """
    t, qh, d = query.shape
    g = qh // num_kv_heads
    q = query.float().view(t, num_kv_heads, g, d).permute(1, 2, 0, 3)
    k = keys.float().unsqueeze(1)
    v = values.float().unsqueeze(1)
    scores = torch.einsum("hgtd,hgnd->hgtn", q, k) * scale
    w = torch.softmax(scores, dim=-1)
    out = torch.einsum("hgtn,hgnd->hgtd", w, v)
    return out.permute(2, 0, 1, 3).reshape(t, qh, d).to(query.dtype)


def hybrid_attention(query: torch.Tensor, planes: Optional[Planes],
                     recent_k: Optional[torch.Tensor], recent_v: Optional[torch.Tensor],
                     num_kv_heads: int, pi: torch.Tensor, s: torch.Tensor,
                     centroids: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
    """compute_hybrid_attention, score.py:29-135: dequantise all history, join
    it with the exact recent tokens, attend once.  History shorter than 16
    tokens is ignored (score.py:26,56); value groups are 32 wide (score.py:94)."""
    t, qh, d = query.shape
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    has_hist = planes is not None and planes.num_tokens >= MIN_HISTORY_FOR_TQ
    has_recent = recent_k is not None and recent_k.shape[0] > 0
    if not has_hist and not has_recent:
        return torch.zeros(t, qh, d, dtype=query.dtype)
    ks, vs = [], []
    if has_hist:
        ks.append(prod_dequantize(planes.mse_indices, planes.qjl_signs, planes.norms,
                                  planes.residual_norms, pi, s, centroids, planes.mse_bits).float())
        vs.append(dequantize_values(planes.v_data, planes.v_scales, planes.v_zeros,
                                    planes.v_bits, 32).float())
    if has_recent:
        ks.append(recent_k.transpose(0, 1).float())
        vs.append(recent_v.transpose(0, 1).float())
    return matmul_attend(query, torch.cat(ks, 1), torch.cat(vs, 1), num_kv_heads, scale)


# --------------------------------------------------------------------------
# synthetic workloads shared by tests and the benchmark
# --------------------------------------------------------------------------

def synth_kv(n_tokens: int, num_kv_heads: int, head_dim: int, seed: int,
             dtype: torch.dtype = torch.float32):
    """Keys N(0,1) x lognormal(0,0.5) per-channel scales, values N(0,1)."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    ch = torch.exp(0.5 * torch.randn(head_dim, generator=g))
    k = torch.randn(n_tokens, num_kv_heads, head_dim, generator=g) * ch
    v = torch.randn(n_tokens, num_kv_heads, head_dim, generator=g)
    return k.to(dtype), v.to(dtype)


def synth_query(n: int, num_q_heads: int, head_dim: int, seed: int,
                dtype: torch.dtype = torch.float32) -> torch.Tensor:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return torch.randn(n, num_q_heads, head_dim, generator=g).to(dtype)

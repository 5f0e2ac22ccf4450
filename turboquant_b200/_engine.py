"""Device-side state shared by the host classes: per-layer constants, block
pools, workspaces, and thin wrappers around the C entry points.

PyTorch is used for device memory and streams only; all arithmetic of the
store and read paths runs in the CUDA library.
"""

from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import torch

from . import _lib
from ._lib import TQ_BF16, TQ_BLOCK_TOKENS, TQ_F16, TQ_F32, check, lib
from .codebook import get_codebook_tensors
from .rotation import generate_qjl_matrix, generate_rotation_matrix

_DTYPES = {torch.float32: TQ_F32, torch.bfloat16: TQ_BF16, torch.float16: TQ_F16}


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt}; use float32, bfloat16 or float16") from None


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: this package has no CPU path")


def get_layout(head_dim: int, key_bits: int, value_bits: int, group_size: int = 32) -> _lib.tq_layout:
    cfg = _lib.tq_config(head_dim, key_bits, value_bits, group_size)
    out = _lib.tq_layout()
    check(lib().tq_get_layout(C.byref(cfg), C.byref(out)), "tq_get_layout")
    return out


def _split_bf16(m: torch.Tensor, n_limbs: int) -> list[torch.Tensor]:
    """m (fp64) as a sum of bf16 limbs, largest first."""
    limbs, rest = [], m.clone()
    for _ in range(n_limbs):
        limb = rest.to(torch.float32).to(torch.bfloat16)
        limbs.append(limb)
        rest = rest - limb.to(torch.float64)
    return limbs


class LayerConstants:
    """Pi, S, the code book and the C struct that carries them (one per layer and shape).

    Seeds follow the reference: Pi from `seed`, S from `seed + 1000`
    (quantizer.py:208), `seed = 42 + 7 * layer_idx` for a layer (store.py:56).
    """

    def __init__(self, head_dim: int, key_bits: int, value_bits: int, device, seed: int = 42,
                 group_size: int = 32, Pi: Optional[torch.Tensor] = None, S: Optional[torch.Tensor] = None,
                 centroids: Optional[torch.Tensor] = None, boundaries: Optional[torch.Tensor] = None,
                 tensor_core_store: bool = True):
        self.head_dim, self.key_bits, self.value_bits = head_dim, key_bits, value_bits
        self.group_size = group_size
        self.device = torch.device(device)
        self.cfg = _lib.tq_config(head_dim, key_bits, value_bits, group_size)
        self.layout = get_layout(head_dim, key_bits, value_bits, group_size)
        mse_bits = key_bits - 1
        pi = generate_rotation_matrix(head_dim, "cpu", seed=seed) if Pi is None else Pi.detach().float().cpu()
        s = generate_qjl_matrix(head_dim, "cpu", seed=seed + 1000) if S is None else S.detach().float().cpu()
        if centroids is None or boundaries is None:
            centroids, boundaries = get_codebook_tensors(head_dim, mse_bits, "cpu")
        self.centroids_cpu = centroids.detach().float().cpu()
        self.boundaries_cpu = boundaries.detach().float().cpu()
        dev = self.device
        self.Pi = pi.contiguous().to(dev)
        self.PiT = pi.T.contiguous().to(dev)
        self.S = s.contiguous().to(dev)
        self.ST = s.T.contiguous().to(dev)
        self.centroids = self.centroids_cpu.to(dev)
        self.boundaries = self.boundaries_cpu.to(dev)
        self.qjl_scale = math.sqrt(math.pi / 2.0) / head_dim
        # operands of the tensor-core store kernel: Pi as three bf16 limbs and
        # M = S Pi^T (the QJL projection applied in rotated space) as two
        m = s.double() @ pi.double().T
        self.pi_limbs = [t.contiguous().to(dev) for t in _split_bf16(pi.double(), 3)]
        self.m_limbs = [t.contiguous().to(dev) for t in _split_bf16(m, 2)]
        # and of the tensor-core query preparation: S as two bf16 limbs (Pi's first two serve there too)
        self.s_limbs = [t.contiguous().to(dev) for t in _split_bf16(s.double(), 2)]

        c = _lib.tq_consts()
        c.cfg = self.cfg
        c.pi, c.pi_t = self.Pi.data_ptr(), self.PiT.data_ptr()
        c.s, c.s_t = self.S.data_ptr(), self.ST.data_ptr()
        n_cent = 1 << mse_bits
        for i in range(n_cent):
            c.centroids[i] = float(self.centroids_cpu[i])
        interior = self.boundaries_cpu[1:-1]
        for i in range(n_cent - 1):
            c.boundaries[i] = float(interior[i])
        c.qjl_scale = self.qjl_scale
        # without the split operands tq_store always runs its fp32 kernel
        for i in range(3):
            c.pi_limbs[i] = self.pi_limbs[i].data_ptr() if tensor_core_store else None
        for i in range(2):
            c.m_limbs[i] = self.m_limbs[i].data_ptr() if tensor_core_store else None
            c.s_limbs[i] = self.s_limbs[i].data_ptr() if tensor_core_store else None
        self.c = c

    @property
    def block_bytes(self) -> int:
        return self.layout.block_bytes

    @property
    def bytes_per_token(self) -> int:
        return self.layout.bytes_per_token


class BlockPool:
    """A pool of block records for `num_kv_heads` heads (uint8 device tensor)."""

    def __init__(self, consts: LayerConstants, num_kv_heads: int, num_blocks: int):
        self.consts = consts
        self.num_kv_heads = num_kv_heads
        self.num_blocks = 0
        self.data = torch.empty(0, dtype=torch.uint8, device=consts.device)
        self.c = _lib.tq_pool()
        self.resize(max(1, num_blocks))

    def resize(self, num_blocks: int) -> None:
        """Grow (never shrink) to `num_blocks`, keeping existing records."""
        if num_blocks <= self.num_blocks:
            return
        per_block = self.num_kv_heads * self.consts.block_bytes
        new = torch.zeros(num_blocks * per_block, dtype=torch.uint8, device=self.consts.device)
        if self.num_blocks:
            new[: self.num_blocks * per_block].copy_(self.data)
        self.data, self.num_blocks = new, num_blocks
        self.c = _lib.tq_pool(self.data.data_ptr(), num_blocks, self.num_kv_heads)

    def nbytes(self) -> int:
        return self.data.numel()

    @classmethod
    def over(cls, consts: LayerConstants, num_kv_heads: int, raw: torch.Tensor) -> "BlockPool":
        """A pool laid over memory somebody else allocated (a serving engine's KV-cache buffer): `raw`
        is a contiguous uint8 device tensor, 16-byte aligned; as many whole blocks as fit are used.
        The pool never grows and never copies."""
        if raw.dtype != torch.uint8 or not raw.is_cuda or not raw.is_contiguous() or raw.data_ptr() % 16:
            raise ValueError("the pool needs a contiguous, 16-byte aligned uint8 device tensor")
        per_block = num_kv_heads * consts.block_bytes
        n = raw.numel() // per_block
        if n < 1:
            raise ValueError(f"{raw.numel()} bytes hold no block of {per_block} bytes")
        pool = cls.__new__(cls)
        pool.consts, pool.num_kv_heads, pool.num_blocks = consts, num_kv_heads, n
        pool.data = raw.view(-1)[: n * per_block]
        pool.c = _lib.tq_pool(pool.data.data_ptr(), n, num_kv_heads)
        pool.resize = pool._fixed
        return pool

    def _fixed(self, num_blocks: int) -> None:
        if num_blocks > self.num_blocks:
            raise RuntimeError(f"a pool over engine memory cannot grow ({self.num_blocks} -> {num_blocks} blocks)")


class Workspace:
    """Zero-initialised scratch for tq_decode / tq_scores; grows on demand."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.buf = torch.empty(0, dtype=torch.uint8, device=self.device)

    def ensure(self, nbytes: int) -> None:
        if self.buf.numel() < nbytes:
            self.buf = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)

    def ensure_decode(self, consts: "LayerConstants", b: int, qh: int, h: int, splits: int) -> None:
        """Size the buffer for one tq_decode shape; the library is asked once per shape."""
        key = (consts.head_dim, consts.key_bits, consts.value_bits, b, qh, h, splits)
        need = _DECODE_WS_BYTES.get(key)
        if need is None:
            n = C.c_size_t(0)
            check(lib().tq_decode_workspace_bytes(C.byref(consts.cfg), b, qh, h, splits, C.byref(n)),
                  "tq_decode_workspace_bytes")
            need = _DECODE_WS_BYTES[key] = n.value
        self.ensure(need)

    @property
    def ptr(self) -> int:
        return self.buf.data_ptr()

    @property
    def nbytes(self) -> int:
        return self.buf.numel()

    def status(self) -> int:
        out = C.c_int32(0)
        check(lib().tq_read_status(self.ptr, stream_ptr(self.device), C.byref(out)), "tq_read_status")
        return out.value


_SM_COUNT: dict[int, int] = {}
_DECODE_WS_BYTES: dict[tuple, int] = {}
_CONST_I32: dict[tuple, torch.Tensor] = {}


def const_i32(device, value: int, n: int = 1) -> torch.Tensor:
    """A cached read-only int32 device tensor of `n` copies of `value` (sequence
    and ring lengths handed to the kernels; small values only are cached)."""
    if not 0 <= value <= 4096 or n > 64:
        return torch.full((n,), value, dtype=torch.int32, device=device)
    key = (str(device), value, n)
    t = _CONST_I32.get(key)
    if t is None:
        t = _CONST_I32[key] = torch.full((n,), value, dtype=torch.int32, device=device)
    return t


def sm_count(device) -> int:
    idx = torch.device(device).index or 0
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


def choose_splits(batch: int, num_kv_heads: int, max_seq_len: int, sms: int, max_ring_len: int = 0) -> int:
    """Sequence splits per (sequence, kv head).  The decode kernel runs one
    12-warp CTA per SM when the launch fits one wave: with few (sequence, head)
    pairs the sequence is cut so that every SM gets one CTA, the ring tokens
    taking CTAs of their own (64 tokens each when the launch fits one wave -
    the library applies the same rule); with many pairs a CTA takes at most
    512 records (8192 tokens) so that long and short sequences balance out."""
    nblk = (max_seq_len + TQ_BLOCK_TOKENS - 1) // TQ_BLOCK_TOKENS
    pairs = max(1, batch * num_kv_heads)
    ring_ctas = (max_ring_len + 63) // 64
    want = max(sms // pairs - ring_ctas, -(-nblk // 512), 1)
    return max(1, min(want, max(1, nblk // 12)))


def store(consts: LayerConstants, pool: BlockPool, key: torch.Tensor, value: torch.Tensor, *,
          stride_token: int, stride_head: int, n_tokens: int, n_heads: int,
          slot_mapping: Optional[torch.Tensor] = None, block_table: Optional[torch.Tensor] = None,
          start_pos: int = 0) -> None:
    require_cuda(key, "key")
    require_cuda(value, "value")
    if key.dtype != value.dtype:
        raise TypeError("key and value must share a dtype")
    check(lib().tq_store(C.byref(consts.c), key.data_ptr(), value.data_ptr(), dtype_code(key.dtype),
                         n_tokens, n_heads, stride_token, stride_head,
                         slot_mapping.data_ptr() if slot_mapping is not None else None,
                         block_table.data_ptr() if block_table is not None else None,
                         start_pos, C.byref(pool.c), stream_ptr(consts.device)), "tq_store")


def store_paged(consts: LayerConstants, pool: BlockPool, key_cache: torch.Tensor, value_cache: torch.Tensor, *,
                src_block_table: torch.Tensor, n_tokens: int, block_table: torch.Tensor, start_pos: int = 0) -> bool:
    """Compress the first n_tokens tokens of a sequence held in a paged cache.

    key_cache / value_cache: (num_blocks, block_size, H, D) views (any block / token / head strides, D
    contiguous, same strides for both); src_block_table: int32 device tensor, logical -> physical block.
    Returns False, with nothing launched, when the call does not fit the table-walking tensor-core
    kernel (the caller then gathers the rows and uses `store`).
    """
    require_cuda(key_cache, "key_cache")
    require_cuda(value_cache, "value_cache")
    if key_cache.dtype != value_cache.dtype or key_cache.shape != value_cache.shape or \
            key_cache.stride() != value_cache.stride() or key_cache.dim() != 4 or key_cache.stride(3) != 1:
        raise ValueError("key_cache and value_cache must be (num_blocks, block_size, H, D) views of one layout")
    if src_block_table.dtype != torch.int32 or not src_block_table.is_cuda or not src_block_table.is_contiguous():
        raise TypeError("src_block_table must be a contiguous int32 device tensor")
    nb, bs, h, _ = key_cache.shape
    if n_tokens > src_block_table.numel() * bs:
        raise ValueError("src_block_table is shorter than n_tokens")
    rc = lib().tq_store_paged(C.byref(consts.c), key_cache.data_ptr(), value_cache.data_ptr(), dtype_code(key_cache.dtype),
                              nb, bs, h, key_cache.stride(0), key_cache.stride(1), key_cache.stride(2),
                              src_block_table.data_ptr(), n_tokens, block_table.data_ptr(), start_pos,
                              C.byref(pool.c), stream_ptr(consts.device))
    if rc == _lib.TQ_ERR_UNSUPPORTED:
        return False
    check(rc, "tq_store_paged")
    return True


def decode(consts: LayerConstants, pool: BlockPool, ws: Workspace, query: torch.Tensor,
           block_table: torch.Tensor, seq_lens: torch.Tensor, max_seq_len: int, *,
           ring_k: Optional[torch.Tensor] = None, ring_v: Optional[torch.Tensor] = None,
           ring_lens: Optional[torch.Tensor] = None, max_ring_len: int = 0,
           ring_stride_seq: int = 0, ring_stride_token: int = 0, scale: Optional[float] = None,
           min_history: int = 16, num_splits: int = 0, out: Optional[torch.Tensor] = None,
           query_prepared: bool = False, kernel: int = 0, static_scratch: bool = False,
           append_k: Optional[torch.Tensor] = None, append_v: Optional[torch.Tensor] = None) -> torch.Tensor:
    """query (B, Qh, D) -> out (B, Qh, D) in the query dtype.

    static_scratch=True routes through tq_decode_static: no workspace tensor is
    touched, the library's built-in scratch array is used (for callers that
    must not allocate); `ws` may then be None.
    """
    require_cuda(query, "query")
    b, qh, d = query.shape
    query = query.contiguous()
    if out is None:
        out = torch.empty_like(query)
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    h = pool.num_kv_heads
    splits = num_splits or choose_splits(b, h, max_seq_len, sm_count(consts.device), max_ring_len)
    if not static_scratch:
        ws.ensure_decode(consts, b, qh, h, splits)
    a = _lib.tq_decode_args()
    a.query, a.q_dtype, a.batch, a.num_q_heads = query.data_ptr(), dtype_code(query.dtype), b, qh
    a.block_table = block_table.data_ptr()
    a.block_table_stride = block_table.stride(0) if block_table.dim() == 2 else block_table.numel()
    a.seq_lens, a.max_seq_len, a.min_history = seq_lens.data_ptr(), max_seq_len, min_history
    if ring_k is not None and max_ring_len > 0:
        a.ring_k, a.ring_v = ring_k.data_ptr(), ring_v.data_ptr()
        a.ring_dtype = dtype_code(ring_k.dtype)
        a.ring_lens, a.max_ring_len = ring_lens.data_ptr(), max_ring_len
        a.ring_stride_seq, a.ring_stride_token = ring_stride_seq, ring_stride_token
    a.scale = scale
    a.out, a.num_splits = out.data_ptr(), splits
    a.query_prepared = 1 if query_prepared else 0
    a.kernel = kernel
    if append_k is not None:      # (B, H, D) new exact token per sequence, appended on the device before attending
        a.append_k, a.append_v = append_k.data_ptr(), append_v.data_ptr()
        a.ring_capacity = ring_k.shape[-3]
    if static_scratch:
        check(lib().tq_decode_static(C.byref(consts.c), C.byref(pool.c), C.byref(a), stream_ptr(consts.device)),
              f"tq_decode_static (built-in scratch of {lib().tq_decode_static_scratch_bytes()} bytes)")
        return out
    a.workspace, a.workspace_bytes = ws.ptr, ws.nbytes
    check(lib().tq_decode(C.byref(consts.c), C.byref(pool.c), C.byref(a), stream_ptr(consts.device)), "tq_decode")
    return out


def scores(consts: LayerConstants, pool: BlockPool, ws: Workspace, block_table: torch.Tensor, n_tokens: int,
           query: torch.Tensor) -> torch.Tensor:
    """query (H, n_q, D) -> unscaled logits (H, n_q, n_tokens) fp32."""
    require_cuda(query, "query")
    h, n_q, d = query.shape
    query = query.contiguous()
    logits = torch.empty(h, n_q, n_tokens, dtype=torch.float32, device=query.device)
    need = C.c_size_t(0)
    check(lib().tq_scores_workspace_bytes(C.byref(consts.cfg), h * n_q, C.byref(need)), "tq_scores_workspace_bytes")
    ws.ensure(need.value)
    check(lib().tq_scores(C.byref(consts.c), C.byref(pool.c), block_table.data_ptr(), n_tokens, query.data_ptr(),
                          dtype_code(query.dtype), n_q, logits.data_ptr(), ws.ptr, ws.nbytes,
                          stream_ptr(consts.device)), "tq_scores")
    return logits


class PlaneSet:
    """Flat planes (H, capacity, ...) on the device plus their C descriptor."""

    def __init__(self, consts: LayerConstants, num_kv_heads: int, capacity: int):
        lay, dev = consts.layout, consts.device
        h, n = num_kv_heads, max(1, capacity)
        self.mse_indices = torch.zeros(h, n, lay.kcode_row, dtype=torch.uint8, device=dev)
        self.qjl_signs = torch.zeros(h, n, lay.ksign_row, dtype=torch.uint8, device=dev)
        self.norms = torch.zeros(h, n, dtype=torch.float16, device=dev)
        self.residual_norms = torch.zeros(h, n, dtype=torch.float16, device=dev)
        self.v_data = torch.zeros(h, n, lay.vcode_row, dtype=torch.uint8, device=dev)
        self.v_scales = torch.zeros(h, n, lay.n_groups, dtype=torch.float16, device=dev)
        self.v_zeros = torch.zeros(h, n, lay.n_groups, dtype=torch.float16, device=dev)
        self.capacity = n
        self.c = _lib.tq_planes(self.mse_indices.data_ptr(), self.qjl_signs.data_ptr(), self.norms.data_ptr(),
                                self.residual_norms.data_ptr(), self.v_data.data_ptr(), self.v_scales.data_ptr(),
                                self.v_zeros.data_ptr(), n)

    @classmethod
    def from_tensors(cls, consts, mse_indices, qjl_signs, norms, residual_norms, v_data, v_scales, v_zeros):
        h, n = mse_indices.shape[0], mse_indices.shape[1]
        ps = cls(consts, h, n)
        dev = consts.device
        ps.mse_indices.copy_(mse_indices.to(dev))
        ps.qjl_signs.copy_(qjl_signs.to(dev))
        ps.norms.copy_(norms.to(dev).to(torch.float16))
        ps.residual_norms.copy_(residual_norms.to(dev).to(torch.float16))
        ps.v_data.copy_(v_data.to(dev))
        ps.v_scales.copy_(v_scales.to(dev).to(torch.float16))
        ps.v_zeros.copy_(v_zeros.to(dev).to(torch.float16))
        return ps


def pool_to_planes(consts: LayerConstants, pool: BlockPool, block_table: torch.Tensor, n_tokens: int) -> PlaneSet:
    ps = PlaneSet(consts, pool.num_kv_heads, n_tokens)
    check(lib().tq_pool_to_planes(C.byref(consts.cfg), C.byref(pool.c), block_table.data_ptr(), n_tokens,
                                  C.byref(ps.c), stream_ptr(consts.device)), "tq_pool_to_planes")
    return ps


def planes_to_pool(consts: LayerConstants, planes: PlaneSet, n_tokens: int, pool: BlockPool,
                   block_table: torch.Tensor, start_pos: int = 0) -> None:
    check(lib().tq_planes_to_pool(C.byref(consts.cfg), C.byref(planes.c), n_tokens, block_table.data_ptr(),
                                  start_pos, C.byref(pool.c), stream_ptr(consts.device)), "tq_planes_to_pool")


def dequant_keys(consts: LayerConstants, pool: BlockPool, block_table: torch.Tensor, n_tokens: int,
                 with_qjl: bool = True) -> torch.Tensor:
    out = torch.empty(pool.num_kv_heads, n_tokens, consts.head_dim, dtype=torch.float32, device=consts.device)
    check(lib().tq_dequant_keys(C.byref(consts.c), C.byref(pool.c), block_table.data_ptr(), n_tokens,
                                1 if with_qjl else 0, out.data_ptr(), stream_ptr(consts.device)), "tq_dequant_keys")
    return out


def dequant_values(consts: LayerConstants, pool: BlockPool, block_table: torch.Tensor, n_tokens: int) -> torch.Tensor:
    out = torch.empty(pool.num_kv_heads, n_tokens, consts.head_dim, dtype=torch.float32, device=consts.device)
    check(lib().tq_dequant_values(C.byref(consts.cfg), C.byref(pool.c), block_table.data_ptr(), n_tokens,
                                  out.data_ptr(), stream_ptr(consts.device)), "tq_dequant_values")
    return out


def identity_block_table(n_blocks: int, device) -> torch.Tensor:
    return torch.arange(max(1, n_blocks), dtype=torch.int32, device=device)


def blocks_for(n_tokens: int) -> int:
    return (n_tokens + TQ_BLOCK_TOKENS - 1) // TQ_BLOCK_TOKENS


def pack_stage(consts: LayerConstants, y: torch.Tensor, projected: torch.Tensor):
    """Integer stages only: rotated vectors -> packed codes, projections -> packed signs."""
    require_cuda(y, "y")
    d = consts.head_dim
    y2 = y.reshape(-1, d).float().contiguous()
    p2 = projected.reshape(-1, d).float().contiguous()
    n = y2.shape[0]
    codes = torch.empty(n, consts.layout.kcode_row, dtype=torch.uint8, device=y.device)
    signs = torch.empty(n, d // 8, dtype=torch.uint8, device=y.device)
    check(lib().tq_pack_stage(C.byref(consts.c), y2.data_ptr(), p2.data_ptr(), n, codes.data_ptr(),
                              signs.data_ptr(), stream_ptr(consts.device)), "tq_pack_stage")
    return codes.reshape(*y.shape[:-1], -1), signs.reshape(*y.shape[:-1], -1)


def prefill_attention_supported(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor) -> bool:
    """Whether `prefill_attention` takes these tensors (CUDA, bf16 / fp16, head_dim 128 or 256, 16-byte
    aligned rows); otherwise the caller keeps its own attention."""
    return (query.is_cuda and key.is_cuda and value.is_cuda and query.dtype in (torch.bfloat16, torch.float16)
            and key.dtype == query.dtype and value.dtype == query.dtype and query.dim() == 3 and key.dim() == 3
            and query.shape[-1] in (128, 256) and key.shape == value.shape and key.shape[-1] == query.shape[-1]
            and query.shape[1] % key.shape[1] == 0 and key.shape[0] == query.shape[0])


def prefill_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, scale: Optional[float] = None,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of a sequence over itself: query (n, Qh, D), key / value (n, H, D) -> (n, Qh, D)."""
    if not prefill_attention_supported(query, key, value):
        raise ValueError("prefill_attention needs CUDA bf16/fp16 tensors (n, heads, 128 or 256)")

    def rows(t):   # D contiguous, 16-byte aligned rows, token stride >= head stride
        ok = t.stride(2) == 1 and t.stride(0) % 8 == 0 and t.stride(1) % 8 == 0 and t.data_ptr() % 16 == 0 \
            and (t.stride(0) >= t.stride(1) or t.shape[1] == 1) and t.stride(1) >= t.shape[2]
        return t if ok else t.contiguous()

    q, k, v = rows(query), rows(key), rows(value)
    if k.stride() != v.stride():
        k, v = k.contiguous(), v.contiguous()
    n, qh, d = q.shape
    if out is None:
        out = torch.empty((n, qh, d), dtype=q.dtype, device=q.device)
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    check(lib().tq_prefill_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dtype_code(q.dtype),
                                     n, qh, k.shape[1], d, q.stride(0), q.stride(1), k.stride(0), k.stride(1),
                                     out.stride(0), out.stride(1), float(scale), stream_ptr(q.device)),
          "tq_prefill_attention")
    return out


def prefill_attention_status() -> int:
    """Status word of the prefill attention kernel (0 = fine); synchronises the device."""
    out = C.c_int32(0)
    check(lib().tq_prefill_attention_read_status(C.byref(out)), "tq_prefill_attention_read_status")
    return out.value


def store_status() -> int:
    """Status word of the tensor-core store kernel (0 = fine); synchronises the device."""
    out = C.c_int32(0)
    check(lib().tq_store_read_status(C.byref(out)), "tq_store_read_status")
    return out.value

"""vLLM adapter: hooks on every attention layer's `do_kv_cache_update` and
`forward`, with the reference's modes and public names (reference
integration/vllm.py:34-528).

    off           nothing is captured, vLLM runs untouched
    capture_only  K/V are compressed into the store, attention stays vLLM's
    hybrid        decode attends over compressed history + exact ring
    full_tq       reserved (as in the reference)

The arithmetic lives in the CUDA library; this file is host plumbing only.
Per-layer device state is created on first use, so installing hooks costs no
GPU memory while the mode is `off`.
"""

from __future__ import annotations

import logging
import math
import types
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.nn.functional as F

from .. import _engine as E
from ..capture import KVCaptureEngine
from ..score import compute_hybrid_attention
from ..store import CompressedKVStore

logger = logging.getLogger("turboquant.integration.vllm")

MODE_OFF = "off"
MODE_CAPTURE_ONLY = "capture_only"
MODE_HYBRID = "hybrid"
MODE_FULL_TQ = "full_tq"
_VALID_MODES = (MODE_OFF, MODE_CAPTURE_ONLY, MODE_HYBRID, MODE_FULL_TQ)
_GLOBAL_MODE = MODE_CAPTURE_ONLY
MIN_HISTORY = 16


def set_mode(mode: str) -> None:
    global _GLOBAL_MODE
    assert mode in _VALID_MODES, f"Invalid mode: {mode}. Valid: {_VALID_MODES}"
    _GLOBAL_MODE = mode
    logger.info("[TurboQuant] Mode set to: %s", mode)


def get_mode() -> str:
    return _GLOBAL_MODE


@dataclass
class LayerConfig:
    head_dim: int
    num_kv_heads: int
    num_query_heads: int
    key_bits: int = 3
    value_bits: int = 2
    value_group_size: int = 32
    ring_capacity: int = 128
    layer_idx: int = 0
    backend_kind: str = "flash"   # "flash" | "mla"
    device: torch.device = field(default_factory=lambda: torch.device("cuda"))


class LayerState:
    """Per-layer runtime state; store and engine appear on first access."""

    def __init__(self, config: LayerConfig):
        self.config = config
        self._store: Optional[CompressedKVStore] = None
        self._engine: Optional[KVCaptureEngine] = None
        self._log_count = 0

    @property
    def store(self) -> CompressedKVStore:
        if self._store is None:
            c = self.config
            self._store = CompressedKVStore(c.head_dim, c.num_kv_heads, c.key_bits, c.value_bits,
                                            c.value_group_size, device=c.device, layer_idx=c.layer_idx)
        return self._store

    @property
    def engine(self) -> KVCaptureEngine:
        if self._engine is None:
            self._engine = KVCaptureEngine(self.store, ring_capacity=self.config.ring_capacity,
                                           device=self.config.device)
        return self._engine

    @property
    def materialized(self) -> bool:
        return self._store is not None

    @property
    def supports_hybrid(self) -> bool:
        return self.config.backend_kind == "flash"

    def reset(self) -> None:
        if self._engine is not None:
            self._engine.reset()
        self._log_count = 0


def _infer_num_query_heads(attn_module, impl) -> int:
    for owner, name in ((attn_module, "num_heads"), (attn_module, "num_attention_heads"), (impl, "num_heads")):
        value = getattr(owner, name, None)
        if value:
            return int(value)
    return int(impl.num_kv_heads)


def _is_mla_impl(impl) -> bool:
    return hasattr(impl, "forward_mqa") and hasattr(impl, "do_kv_cache_update") and not hasattr(impl, "forward")


def _capture(state: LayerState, key, value, num_tokens: int) -> None:
    """One token goes to the ring, a longer run is a prefill (reference vllm.py:139-145)."""
    if num_tokens <= 1:
        state.engine.ingest_decode(key, value, num_tokens)
    else:
        state.engine.ingest_prefill(key, value, num_tokens)


def _as_heads(t: torch.Tensor, n: int, heads: int, dim: int) -> torch.Tensor:
    t = t[:n]
    return t.view(n, heads, dim) if t.dim() == 2 else t


def _deliver(result: torch.Tensor, query: torch.Tensor, output, n: int):
    """Hand `result` (n, Qh, D) back the way vLLM expects it."""
    flat = result.reshape(n, -1).to(query.dtype)
    if output is not None:
        dst = output[:n]
        dst.copy_(result.to(dst.dtype) if dst.dim() == 3 else flat.to(dst.dtype))
        return output
    return result.to(query.dtype) if query.dim() == 3 else flat


def _no_alloc_prefill_attention(state: LayerState, impl, query, key, value, attn_metadata) -> torch.Tensor:
    """Causal prefill attention from the layer's own K/V when no paged cache exists (reference
    vllm.py:150-180).  16-bit CUDA tensors with head_dim 128 / 256 go through the library's tensor-core
    kernel, which reads each kv head in place for its group of query heads (no repeat_interleave) and
    lets the store of the same K/V, launched next on the stream, begin under its tail; anything else
    takes torch's attention like the reference."""
    c = state.config
    n = attn_metadata.num_actual_tokens
    q = _as_heads(query, n, c.num_query_heads, c.head_dim)
    k = _as_heads(key, n, c.num_kv_heads, c.head_dim)
    v = _as_heads(value, n, c.num_kv_heads, c.head_dim)
    scale = getattr(impl, "scale", 1.0 / math.sqrt(c.head_dim))
    if E.prefill_attention_supported(q, k, v):
        return E.prefill_attention(q, k, v, scale=scale)
    rep = c.num_query_heads // c.num_kv_heads
    if rep > 1:
        k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    out = F.scaled_dot_product_attention(q.transpose(0, 1).unsqueeze(0), k.transpose(0, 1).unsqueeze(0),
                                         v.transpose(0, 1).unsqueeze(0), is_causal=True, scale=scale)
    return out.squeeze(0).transpose(0, 1)


def _make_patched_kv_update(orig_fn, state: LayerState, no_alloc: bool = False):
    def patched(self_impl, layer, key, value, kv_cache, slot_mapping):
        if not no_alloc:
            orig_fn(self_impl, layer, key, value, kv_cache, slot_mapping)
        if _GLOBAL_MODE != MODE_OFF:
            _capture(state, key, value, slot_mapping.shape[0])
    return patched


def _make_patched_forward(orig_fn, state: LayerState, no_alloc: bool = False, capture_in_forward: bool = False):
    def original(self_impl, layer, query, key, value, kv_cache, md, output, output_scale, output_block_scale):
        return orig_fn(self_impl, layer, query, key, value, kv_cache, md, output, output_scale, output_block_scale)

    def patched(self_impl, layer, query, key, value, kv_cache, attn_metadata, output=None, output_scale=None,
                output_block_scale=None):
        mode = _GLOBAL_MODE
        args = (self_impl, layer, query, key, value, kv_cache, attn_metadata, output, output_scale,
                output_block_scale)
        if capture_in_forward and mode != MODE_OFF and attn_metadata is not None:
            n = getattr(attn_metadata, "num_actual_tokens", key.shape[0])
            c = state.config
            if (mode == MODE_HYBRID and n == 1 and getattr(attn_metadata, "max_query_len", 1) == 1
                    and state.supports_hybrid and state.store.num_tokens >= MIN_HISTORY
                    and key.dtype == state.engine.ring.dtype and query.dtype == key.dtype):
                # one decode token: ring append and attention in ONE library call, same result as
                # capturing first and attending afterwards
                result = state.engine.decode_step(_as_heads(query, 1, c.num_query_heads, c.head_dim),
                                                  _as_heads(key, 1, c.num_kv_heads, c.head_dim),
                                                  _as_heads(value, 1, c.num_kv_heads, c.head_dim),
                                                  c.num_query_heads, scale=getattr(self_impl, "scale", None))
                return _deliver(result, query, output, 1)
            _capture(state, key[:n], value[:n], n)
        if mode in (MODE_OFF, MODE_CAPTURE_ONLY) or attn_metadata is None:
            return original(*args)
        c = state.config
        n = attn_metadata.num_actual_tokens
        if attn_metadata.max_query_len > 1:            # prefill
            if not no_alloc:
                return original(*args)
            return _deliver(_no_alloc_prefill_attention(state, self_impl, query, key, value, attn_metadata),
                            query, output, n)
        if mode == MODE_HYBRID and state.supports_hybrid and state.store.num_tokens >= MIN_HISTORY:
            q = _as_heads(query, n, c.num_query_heads, c.head_dim)
            recent = state.engine.ring.peek()
            result = compute_hybrid_attention(q, state.store, recent[0] if recent else None,
                                              recent[1] if recent else None, c.num_query_heads,
                                              scale=getattr(self_impl, "scale", None))
            return _deliver(result, query, output, n)
        if no_alloc:                                    # nothing to attend to yet and no paged cache to fall back on
            shape = (n, c.num_query_heads, c.head_dim) if query.dim() == 3 else (n, c.num_query_heads * c.head_dim)
            return torch.zeros(shape, dtype=query.dtype, device=query.device)
        return original(*args)

    return patched


def _bind(impl, name: str, fn) -> None:
    setattr(impl, name, types.MethodType(lambda self, *a, _f=fn, **kw: _f(self, *a, **kw), impl))


def install_hooks(model_runner, key_bits: int = 3, value_bits: int = 2, value_group_size: int = 32,
                  ring_capacity: int = 128, initial_layers_count: int = 4,
                  initial_layers_key_bits: Optional[int] = None, mode: str = MODE_CAPTURE_ONLY,
                  no_alloc: bool = False) -> dict:
    """Hook every attention layer of a vLLM model runner; returns {layer name: LayerState}.

    The first `initial_layers_count` layers get one more key bit (capped at 4),
    as in the reference (vllm.py:358-359,383).  MLA layers are left untouched.
    """
    set_mode(mode)
    if initial_layers_key_bits is None:
        initial_layers_key_bits = min(key_bits + 1, 4)
    states: dict[str, LayerState] = {}
    idx = 0
    for name, module in model_runner.compilation_config.static_forward_context.items():
        impl = getattr(module, "impl", None)
        if impl is None or getattr(impl, "num_kv_heads", None) is None:
            continue
        if hasattr(impl, "head_size"):
            head_dim = int(impl.head_size)
        elif hasattr(impl, "kv_lora_rank"):
            head_dim = int(impl.kv_lora_rank)
        else:
            continue
        kind = "mla" if _is_mla_impl(impl) else "flash"
        cfg = LayerConfig(head_dim=head_dim, num_kv_heads=int(impl.num_kv_heads),
                          num_query_heads=_infer_num_query_heads(module, impl),
                          key_bits=initial_layers_key_bits if idx < initial_layers_count else key_bits,
                          value_bits=value_bits, value_group_size=min(value_group_size, head_dim),
                          ring_capacity=ring_capacity, layer_idx=idx, backend_kind=kind,
                          device=model_runner.device)
        state = LayerState(cfg)
        states[name] = state
        if kind == "flash":
            separate_update = hasattr(impl, "do_kv_cache_update")
            if separate_update:
                _bind(impl, "do_kv_cache_update",
                      _make_patched_kv_update(impl.do_kv_cache_update.__func__, state, no_alloc=no_alloc))
            _bind(impl, "forward", _make_patched_forward(impl.forward.__func__, state, no_alloc=no_alloc,
                                                         capture_in_forward=not separate_update))
        impl._tq_layer_state = state
        idx += 1
    model_runner._tq_layer_states = states
    model_runner._tq_no_alloc = no_alloc
    logger.info("[TurboQuant] Hooks on %d layers (mode=%s, no_alloc=%s)", len(states), mode, no_alloc)
    return states


def free_kv_cache(model_runner) -> int:
    """Replace the paged bf16 KV tensors of hooked (non-MLA) layers by a 1-byte
    tensor; returns the bytes released (reference vllm.py:452-501)."""
    states = getattr(model_runner, "_tq_layer_states", None)
    if not states:
        return 0
    ctx = model_runner.compilation_config.static_forward_context
    tiny = torch.zeros(1, dtype=torch.int8, device=model_runner.device)
    freed, gone = 0, set()
    for name, state in states.items():
        kv_list = getattr(ctx.get(name), "kv_cache", None) if state.supports_hybrid else None
        if kv_list:
            old = kv_list[0]
            gone.add(old.data_ptr())
            freed += old.nelement() * old.element_size()
            kv_list[0] = tiny
    caches = getattr(model_runner, "kv_caches", [])
    for i, entry in enumerate(caches):
        if isinstance(entry, list):
            for j, t in enumerate(entry):
                if hasattr(t, "data_ptr") and t.data_ptr() in gone:
                    entry[j] = tiny
        elif hasattr(entry, "data_ptr") and entry.data_ptr() in gone:
            caches[i] = tiny
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    return freed


def compressed_cache_specs(model_runner) -> dict:
    """Page geometry per hooked attention layer, for an engine that allocates its KV block pool at COMPRESSED
    size instead of allocating bf16 pages first and dropping them with `free_kv_cache` (reference
    vllm.py:452-501).  {layer name: CompressedCacheSpec}; MLA layers, which the hooks leave alone, are absent.
    The engine sizes its pool with `spec.page_size_bytes`, hands each layer's buffer to
    `CompressedPagedKVCache(spec, raw, layer_idx)` and then writes with its slot mappings and reads with its
    block tables."""
    from ..paged_cache import kv_cache_specs
    return kv_cache_specs(getattr(model_runner, "_tq_layer_states", None) or {})


def get_stats(model_runner) -> dict:
    states = getattr(model_runner, "_tq_layer_states", None)
    if not states:
        return {}
    live = [s for s in states.values() if s.materialized]
    n = max(len(states), 1)
    return {"num_layers": len(states),
            "total_compressed_tokens": sum(s.store.num_tokens for s in live) // n,
            "total_buffered_tokens": sum(s.engine.ring.size for s in live) // n,
            "total_memory_bytes": sum(s.store.memory_bytes() for s in live),
            "mode": _GLOBAL_MODE}

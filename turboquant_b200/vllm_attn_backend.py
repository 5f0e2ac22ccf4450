"""Legacy-named entry points of the vLLM adapter (reference vllm_attn_backend.py:17-264):
the older mode names map onto the adapter's modes.

    shadow      -> capture_only   (compress alongside vLLM's cache, never used for output)
    accumulate  -> capture_only
    active      -> hybrid         (decode reads the compressed store)
"""

from __future__ import annotations

from .integration import vllm as _v

MODE_SHADOW = "shadow"
MODE_ACCUMULATE = "accumulate"
MODE_ACTIVE = "active"
_LEGACY = {MODE_SHADOW: _v.MODE_CAPTURE_ONLY, MODE_ACCUMULATE: _v.MODE_CAPTURE_ONLY, MODE_ACTIVE: _v.MODE_HYBRID}
_CURRENT = MODE_ACCUMULATE


def set_mode(mode: str) -> None:
    global _CURRENT
    if mode not in _LEGACY:
        raise ValueError(f"unknown mode {mode!r}; expected one of {sorted(_LEGACY)}")
    _CURRENT = mode
    _v.set_mode(_LEGACY[mode])


def get_mode() -> str:
    return _CURRENT


def install_turboquant_hooks(model_runner, key_bits: int = 3, value_bits: int = 2, value_group_size: int = 32,
                             buffer_size: int = 128, initial_layers_count: int = 4,
                             initial_layers_key_bits=None, mode: str = MODE_ACCUMULATE, no_alloc: bool = False):
    """Install the hooks with the legacy argument names; returns {layer name: LayerState}."""
    global _CURRENT
    if mode not in _LEGACY:
        raise ValueError(f"unknown mode {mode!r}; expected one of {sorted(_LEGACY)}")
    _CURRENT = mode
    return _v.install_hooks(model_runner, key_bits=key_bits, value_bits=value_bits,
                            value_group_size=value_group_size, ring_capacity=buffer_size,
                            initial_layers_count=initial_layers_count,
                            initial_layers_key_bits=initial_layers_key_bits, mode=_LEGACY[mode], no_alloc=no_alloc)


def free_kv_cache(model_runner) -> int:
    return _v.free_kv_cache(model_runner)


def enable_no_alloc(*args, **kwargs):
    """The reference patches vLLM's executor so that hooked layers get no paged
    cache at all (vllm_attn_backend.py:77-214); that is engine plumbing tied to
    one vLLM version and is not part of this package.  Pass `no_alloc=True` to
    install_turboquant_hooks and size the engine's cache yourself."""
    raise NotImplementedError("executor patching is outside this package; use no_alloc=True on the hooks")

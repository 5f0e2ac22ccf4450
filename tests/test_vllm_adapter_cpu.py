"""vLLM adapter host logic with a fake model runner (no GPU, no vLLM import):
hook installation, layer configuration rules, mode switching, pass-through."""

import types

import pytest
import torch

from turboquant_b200 import vllm_attn_backend as legacy
from turboquant_b200.integration import vllm as adapter


class FakeImpl:
    def __init__(self, num_kv_heads=2, head_size=128, num_heads=8):
        self.num_kv_heads, self.head_size, self.num_heads, self.scale = num_kv_heads, head_size, num_heads, 0.1
        self.calls = []

    def do_kv_cache_update(self, layer, key, value, kv_cache, slot_mapping):
        self.calls.append(("update", key.shape[0]))

    def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None, output_scale=None,
                output_block_scale=None):
        self.calls.append(("forward", query.shape[0]))
        return "flash-output"


class FakeMLAImpl:
    num_kv_heads, kv_lora_rank = 1, 512

    def forward_mqa(self, *a):
        return "mla"

    def do_kv_cache_update(self, *a):
        return None


def _runner(n_layers=6):
    ctx = {f"layers.{i}.attn": types.SimpleNamespace(impl=FakeImpl(), num_heads=8) for i in range(n_layers)}
    ctx["layers.mla"] = types.SimpleNamespace(impl=FakeMLAImpl())
    ctx["norm"] = types.SimpleNamespace()          # no impl: skipped
    return types.SimpleNamespace(compilation_config=types.SimpleNamespace(static_forward_context=ctx),
                                 device=torch.device("cpu"), kv_caches=[])


def test_install_configures_layers_like_the_reference():
    r = _runner()
    states = adapter.install_hooks(r, key_bits=3, value_bits=2, ring_capacity=64, mode=adapter.MODE_OFF)
    assert len(states) == 7 and r._tq_layer_states is states
    cfgs = [s.config for s in states.values()]
    assert [c.key_bits for c in cfgs[:6]] == [4, 4, 4, 4, 3, 3]          # first four layers get one more bit
    assert [c.layer_idx for c in cfgs] == list(range(7))
    assert cfgs[0].num_query_heads == 8 and cfgs[0].ring_capacity == 64 and cfgs[0].backend_kind == "flash"
    assert cfgs[6].backend_kind == "mla" and cfgs[6].head_dim == 512 and not states["layers.mla"].supports_hybrid
    assert not any(s.materialized for s in states.values())              # no device state until used


def test_off_and_capture_only_pass_through_without_touching_the_gpu():
    r = _runner(1)
    states = adapter.install_hooks(r, mode=adapter.MODE_OFF)
    impl = r.compilation_config.static_forward_context["layers.0.attn"].impl
    k = torch.zeros(5, 2, 128)
    impl.do_kv_cache_update(None, k, k, None, torch.zeros(5, dtype=torch.long))
    md = types.SimpleNamespace(num_actual_tokens=5, max_query_len=5)
    assert impl.forward(None, torch.zeros(5, 8, 128), k, k, None, md) == "flash-output"
    assert impl.calls == [("update", 5), ("forward", 5)]
    assert not states["layers.0.attn"].materialized
    assert adapter.get_stats(r)["total_compressed_tokens"] == 0 and adapter.get_stats(r)["mode"] == "off"


def test_modes():
    adapter.set_mode(adapter.MODE_HYBRID)
    assert adapter.get_mode() == "hybrid"
    with pytest.raises(AssertionError):
        adapter.set_mode("nonsense")
    legacy.set_mode(legacy.MODE_ACTIVE)
    assert legacy.get_mode() == "active" and adapter.get_mode() == adapter.MODE_HYBRID
    legacy.set_mode(legacy.MODE_SHADOW)
    assert adapter.get_mode() == adapter.MODE_CAPTURE_ONLY
    with pytest.raises(ValueError):
        legacy.set_mode("hybrid")
    with pytest.raises(NotImplementedError):
        legacy.enable_no_alloc()
    adapter.set_mode(adapter.MODE_OFF)


def test_free_kv_cache_swaps_hooked_layers_only():
    r = _runner(2)
    adapter.install_hooks(r, mode=adapter.MODE_OFF)
    ctx = r.compilation_config.static_forward_context
    big = [torch.zeros(2, 4, 16, 2, 128, dtype=torch.bfloat16) for _ in range(3)]
    ctx["layers.0.attn"].kv_cache = [big[0]]
    ctx["layers.1.attn"].kv_cache = [big[1]]
    ctx["layers.mla"].kv_cache = [big[2]]
    r.kv_caches = [big[0], [big[1]], big[2]]
    freed = adapter.free_kv_cache(r)
    assert freed == 2 * big[0].numel() * 2
    assert ctx["layers.0.attn"].kv_cache[0].numel() == 1 and ctx["layers.mla"].kv_cache[0] is big[2]
    assert r.kv_caches[0].numel() == 1 and r.kv_caches[1][0].numel() == 1 and r.kv_caches[2] is big[2]


def test_compressed_cache_specs_follow_the_layer_configuration():
    """The engine-facing page specs: one per hooked flash layer, with that layer's bit widths (the first
    layers keep one more key bit), none for MLA layers; a page of 16 tokens x 2 kv heads."""
    r = _runner(6)
    adapter.install_hooks(r, key_bits=3, value_bits=2, mode=adapter.MODE_OFF)
    specs = adapter.compressed_cache_specs(r)
    assert sorted(specs) == [f"layers.{i}.attn" for i in range(6)]
    assert [specs[f"layers.{i}.attn"].key_bits for i in range(6)] == [4, 4, 4, 4, 3, 3]
    s = specs["layers.5.attn"]
    assert (s.head_dim, s.num_kv_heads, s.page_size_bytes) == (128, 2, 16 * 2 * 100)
    assert specs["layers.0.attn"].page_size_bytes == 16 * 2 * 132      # 4-bit keys: 3-bit codes in nibbles, 32 bytes more per token
    assert adapter.compressed_cache_specs(types.SimpleNamespace()) == {}

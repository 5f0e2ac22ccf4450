"""The CPU oracle against the golden vectors produced by the reference.

Integer stages fed the reference's own fp32 intermediates must match to the
bit.  Stages that go through a GEMM or a norm on this machine's CPU may differ
from the fixture (made on another CPU) in the last bit of a float, which can
flip a code only at a decision-boundary tie: at most 0.01 % of codes.
"""

import numpy as np
import torch

from oracle import tq_oracle as O

TIE_BUDGET = 1e-4  # fraction of codes that may differ end to end


def _frac_diff(a, b):
    a = np.asarray(a)
    b = np.asarray(b)
    assert a.shape == b.shape
    return float((a != b).mean())


def test_bucket_and_pack_bit_exact(golden):
    interior = golden.boundaries[1:-1].numpy()
    idx = O.bucket_indices(golden.y.numpy(), interior)
    packed = O.pack_indices(idx, golden.mse_bits)
    assert np.array_equal(packed, golden.mse_indices.numpy())
    assert np.array_equal(O.unpack_indices(packed, golden.mse_bits, golden.D), idx)


def test_sign_pack_bit_exact(golden):
    signs = O.pack_signs(golden.projected.numpy())
    assert np.array_equal(signs, golden.qjl_signs.numpy())
    sg = O.unpack_signs(signs, golden.D)
    assert set(np.unique(sg)) <= {-1.0, 1.0}


def test_key_path_end_to_end(golden):
    k = golden.key[:golden.T].transpose(0, 1)
    st = O.prod_quantize(k, golden.Pi, golden.S, golden.centroids, golden.boundaries, golden.key_bits)
    assert torch.equal(st.norms, golden.norms)
    assert torch.equal(st.x_unit, golden.x_unit)
    assert _frac_diff(st.packed, golden.mse_indices.numpy()) <= TIE_BUDGET
    assert _frac_diff(st.signs, golden.qjl_signs.numpy()) <= TIE_BUDGET
    torch.testing.assert_close(st.residual_norms, golden.residual_norms, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(st.y, golden.y, rtol=0, atol=1e-6)


def test_value_path_bit_exact(golden):
    v = golden.value[:golden.T].transpose(0, 1)
    data, scales, zeros = O.quantize_values(v, golden.value_bits, 32)
    assert np.array_equal(data, golden.v_data.numpy())
    assert torch.equal(scales, golden.v_scales)
    assert torch.equal(zeros, golden.v_zeros)
    deq = O.dequantize_values(data, scales, zeros, golden.value_bits)
    assert deq.shape == v.shape


def test_store_chunks_and_memory_bytes(golden):
    st = O.OracleStore(golden.D, golden.H, golden.key_bits, golden.value_bits,
                       golden.centroids, golden.boundaries, pi=golden.Pi, s=golden.S)
    t0 = (golden.T * 2) // 3
    st.append_chunk(golden.key[:t0], golden.value[:t0])
    st.append_chunk(golden.key[t0:golden.T], golden.value[t0:golden.T])
    flat = st.get_flat_cache()
    assert flat.num_tokens == golden.T
    assert flat.memory_bytes() == golden.memory_bytes
    assert _frac_diff(flat.mse_indices, golden.mse_indices.numpy()) <= TIE_BUDGET
    assert np.array_equal(flat.v_data, golden.v_data.numpy())


def _planes(golden):
    return O.Planes(golden.mse_indices.numpy(), golden.qjl_signs.numpy(), golden.norms,
                    golden.residual_norms, golden.v_data.numpy(), golden.v_scales, golden.v_zeros,
                    golden.mse_bits, golden.value_bits)


def test_scores_and_dequant(golden):
    p = _planes(golden)
    q = golden.query.float().view(3, golden.H, golden.Qh // golden.H, golden.D)
    q = q.permute(1, 2, 0, 3).reshape(golden.H, -1, golden.D)
    logits = O.attention_score(q, p.mse_indices, p.qjl_signs, p.norms, p.residual_norms,
                               golden.Pi, golden.S, golden.centroids, golden.mse_bits)
    ref = golden.logits
    assert float((logits - ref).abs().max() / ref.abs().max()) < 1e-5
    kd = O.prod_dequantize(p.mse_indices, p.qjl_signs, p.norms, p.residual_norms,
                           golden.Pi, golden.S, golden.centroids, golden.mse_bits)
    torch.testing.assert_close(kd.float(), golden.k_dequant, rtol=1e-4, atol=1e-5)


def test_hybrid_attention(golden):
    p = _planes(golden)
    rk, rv = golden.key[golden.T:], golden.value[golden.T:]
    out = O.hybrid_attention(golden.query, p, rk, rv, golden.H, golden.Pi, golden.S, golden.centroids)
    assert out.dtype == golden.dtype
    cos = torch.nn.functional.cosine_similarity(out.float().flatten(), golden.out_hybrid.float().flatten(), dim=0)
    assert float(cos) > 0.99999
    out_h = O.hybrid_attention(golden.query, p, None, None, golden.H, golden.Pi, golden.S, golden.centroids)
    torch.testing.assert_close(out_h.float(), golden.out_hist.float(), rtol=2e-2, atol=2e-3)


def test_short_history_is_ignored():
    g = __import__("tests.conftest", fromlist=["load_golden"]).load_golden("d128_bf16_k3v2")
    p = _planes(g)
    short = O.Planes(p.mse_indices[:, :15], p.qjl_signs[:, :15], p.norms[:, :15], p.residual_norms[:, :15],
                     p.v_data[:, :15], p.v_scales[:, :15], p.v_zeros[:, :15], p.mse_bits, p.v_bits)
    out = O.hybrid_attention(g.query, short, None, None, g.H, g.Pi, g.S, g.centroids)
    assert float(out.float().abs().max()) == 0.0


def test_constants_follow_reference_seeds():
    g = __import__("tests.conftest", fromlist=["load_golden"]).load_golden("d128_bf16_k3v2")
    seed_pi, seed_s = O.layer_seeds(g.layer)
    assert torch.equal(O.qjl_matrix(g.D, seed_s), g.S)
    pi = O.rotation_matrix(g.D, seed_pi)
    torch.testing.assert_close(pi, g.Pi, rtol=0, atol=1e-5)
    eye = pi @ pi.T
    torch.testing.assert_close(eye, torch.eye(g.D), rtol=0, atol=1e-5)

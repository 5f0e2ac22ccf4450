"""CPU emulation of the arithmetic short-cuts of the tensor-core store kernel
(csrc/tq_store_tc.cu), step by step in numpy / torch, against the oracle's
restatement of the reference (quantizer.py:129-149,231-257, kv_cache.py:45-98).

The kernel replaces three things the reference does in bf16 tensors:
  1. x / d rounded to bf16  ->  bf16(x * fp32(1/d)), no division;
  2. round-half-even + clamp of a bf16 value in [0, 16)  ->  one bf16 addition of 128;
  3. the residual x - x_hat  ->  (Y - c) + E in rotated space, scaled by |x| afterwards.
1 and 2 must be bit-identical, 3 must stay within the tie budget (1e-4 of codes / sign bits).
"""

import numpy as np
import pytest
import torch

from oracle import tq_oracle as O
from turboquant_b200.codebook import get_codebook_tensors


def bf16(x: np.ndarray) -> np.ndarray:
    """fp32 -> nearest bf16 (ties to even) -> fp32, as cvt.rn.bf16.f32 does."""
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(torch.bfloat16).float().numpy()


def all_positive_bf16(lo_exp=-20, hi_exp=20) -> np.ndarray:
    mant = np.arange(128, 256, dtype=np.float64) / 128.0
    return np.concatenate([mant * 2.0 ** e for e in range(lo_exp, hi_exp + 1)]).astype(np.float32)


def test_bf16_quotient_equals_product_with_fp32_reciprocal():
    """Every pair of bf16 significands over a span of exponents: bf16(fl32(a / b)) == bf16(a * fl32(1 / b)).
    The quotient of two 8-bit significands is either a dyadic number with at most 8 bits (exact in bf16)
    or at least 2^-17 away from every bf16 rounding boundary, far more than the reciprocal's error."""
    a_sig = (np.arange(128, 256, dtype=np.float32) / 128.0)
    worst = 1.0
    for ea in (-9, -3, 0, 1, 6):
        a = (a_sig * np.float32(2.0 ** ea))[:, None]
        for eb in (-30, -5, 0, 2, 11):
            b = (a_sig * np.float32(2.0 ** eb))[None, :]
            exact = bf16((a / b).astype(np.float32))
            fast = bf16(a * (np.float32(1.0) / b).astype(np.float32))
            assert np.array_equal(exact, fast), (ea, eb)
            # distance of the true quotient to the nearest rounding boundary, in units of the quotient
            qd = a.astype(np.float64) / b.astype(np.float64)
            m, _ = np.frexp(qd)                      # qd = m * 2^e, m in [0.5, 1): bf16 spacing 2^-8 * 2^e... in m: 2^-8
            frac = (m * 256.0) % 1.0                 # position between two bf16 neighbours
            off = np.abs(frac - 0.5)
            off = off[(frac != 0.0)]                 # exactly representable quotients are nowhere near a tie
            worst = min(worst, float(off.min()))
    assert worst * 2.0 ** -8 > 2.0 ** -17            # margin versus ~2^-23 of rounding error in the product


@pytest.mark.parametrize("levels", [3, 15])
def test_adding_128_in_bf16_is_round_half_even(levels):
    """bf16(z + 128) has unit spacing, so its low mantissa bits are rint(z) for 0 <= z < 128."""
    z = all_positive_bf16(-24, 4)
    z = np.concatenate([[0.0], z[z <= levels + 0.6]]).astype(np.float32)
    zc = np.minimum(z, np.float32(levels))
    summed = bf16(zc + np.float32(128.0))            # z + 128 is exact in fp32 or nowhere near a bf16 tie
    code = (summed.view(np.uint32) >> 16) & (0xF if levels == 15 else 0x3)
    want = np.clip(np.rint(z), 0, levels).astype(np.uint32)
    assert np.array_equal(code, want)


def kernel_value_quant(v_bf16: torch.Tensor, bits: int):
    """quantize_value_group of the kernel on (..., 32) groups, fp32 numpy holding bf16 values."""
    n = float(2 ** bits - 1)
    v = v_bf16.float().numpy()
    vmin, vmax = v.min(-1, keepdims=True), v.max(-1, keepdims=True)
    scale = bf16(bf16(vmax - vmin) / np.float32(n))
    scale = np.maximum(scale, bf16(np.float32(1e-10)))
    rscale = (np.float32(1.0) / scale).astype(np.float32)
    d = bf16(v - vmin)                               # packed bf16 subtraction: one rounding
    z = np.minimum(bf16(d * rscale), np.float32(n))
    code = (bf16(z + np.float32(128.0)).view(np.uint32) >> 16) & int(n)
    return code.astype(np.uint8), scale[..., 0], vmin[..., 0]


@pytest.mark.parametrize("bits", [2, 4])
def test_value_quantisation_short_cuts_are_bit_exact(bits):
    g = torch.Generator().manual_seed(5 + bits)
    v = torch.randn(4096, 8, 128, generator=g)
    v[0, 0, :32] = 0.25                              # constant group
    v[1, 0, :32] = torch.linspace(-3, 3, 32)         # ties at exact thirds / fifteenths
    v[2] *= 1e-6
    v[3] *= 300.0
    v = v.to(torch.bfloat16)
    data, scales, zeros = O.quantize_values(v, bits, 32)
    code, sc, zr = kernel_value_quant(v.reshape(4096, 8, 4, 32), bits)
    assert np.array_equal(O.pack_values(code.reshape(4096, 8, 128), bits), data)
    assert np.array_equal(sc, scales.float().numpy()) and np.array_equal(zr, zeros.float().numpy())


def split_bf16(m: torch.Tensor, n: int):
    out, rest = [], m.double().clone()
    for _ in range(n):
        limb = rest.float().to(torch.bfloat16)
        out.append(limb.float())
        rest = rest - limb.double()
    return out


@pytest.mark.parametrize("d,key_bits", [(128, 3), (128, 4), (256, 3)])
def test_rotated_space_residual_stays_within_the_tie_budget(d, key_bits):
    """The kernel's key path - u = bf16(x * 1/|x|), e' = x/|x| - u as bf16, Y = u (Pi_hi + Pi_lo)^T,
    E = e' Pi_hi^T, r' = (Y - c) + E as bf16 hi + lo, P = r' M^T with M = S Pi^T in two limbs - against
    the oracle: codes and sign bits within 1e-4, norms equal, residual norms within 1e-3."""
    h, n = 8, 8192
    k, _ = O.synth_kv(n, h, d, seed=1003, dtype=torch.bfloat16)
    cent, bnd = get_codebook_tensors(d, key_bits - 1, "cpu")
    pi, s = O.rotation_matrix(d, 42), O.qjl_matrix(d, 1042)
    x = k.transpose(0, 1).reshape(-1, d)
    ref = O.prod_quantize(x, pi, s, cent, bnd, key_bits)

    xf = x.float().numpy()
    nd = bf16(np.sqrt((xf.astype(np.float32) ** 2).sum(-1, dtype=np.float32)))[:, None]
    den = bf16(nd + np.float32(1e-10))
    q = xf * (np.float32(1.0) / den).astype(np.float32)
    u = bf16(q)
    ep = bf16(q - u)
    pl = split_bf16(pi, 2)
    ml = split_bf16(s.double() @ pi.double().T, 2)
    ut, et = torch.from_numpy(u), torch.from_numpy(ep)
    y = ut @ pl[0].T + ut @ pl[1].T
    e = et @ pl[0].T
    idx = O.bucket_indices(y.numpy(), bnd[1:-1].numpy())
    assert float((idx != ref.idx).mean()) <= 1e-4
    r = (y - cent[torch.from_numpy(idx.astype(np.int64))]) + e
    rh = r.to(torch.bfloat16).float()
    rl = (r - rh).to(torch.bfloat16).float()
    p = rh @ ml[0].T + rh @ ml[1].T + rl @ ml[0].T
    signs = O.pack_signs(p.numpy())
    assert float(np.unpackbits(signs ^ ref.signs).sum()) / (signs.size * 8) <= 1e-4
    assert float((torch.from_numpy(nd[:, 0]) != ref.norms.float()).float().mean()) <= 1e-4
    rnorm = torch.from_numpy(nd[:, 0]) * r.norm(dim=-1)
    assert float(((rnorm - ref.residual_norms).abs() / ref.residual_norms).max()) <= 1e-3

"""The C-ABI library without a GPU: it loads, exports every declared symbol,
answers host-only queries and validates arguments before touching CUDA."""

import ctypes as C
import os
import re

import numpy as np
import pytest

from turboquant_b200 import _lib
from turboquant_b200.build import LIB_PATH, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(LIB_PATH):
        build()
    return _lib.lib()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "turboquant_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tq_[a-z_0-9]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = _declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), n
    assert set(names) == set(_lib.SIGNATURES), "binding table and header disagree"


@pytest.mark.parametrize("d,kb,vb,bpt", [(128, 3, 2, 100), (256, 3, 2, 196), (128, 4, 4, 164), (256, 4, 4, 324)])
def test_layout_matches_reference_byte_accounting(lib, d, kb, vb, bpt):
    cfg = _lib.tq_config(d, kb, vb, 32)
    lay = _lib.tq_layout()
    assert lib.tq_get_layout(C.byref(cfg), C.byref(lay)) == 0
    assert lay.bytes_per_token == bpt and lay.block_bytes == 16 * bpt
    offs = [lay.off_kcodes, lay.off_ksigns, lay.off_knorm, lay.off_krnorm, lay.off_vcodes, lay.off_vscale,
            lay.off_vzero, lay.block_bytes]
    assert offs == sorted(offs) and all(o % 16 == 0 for o in offs)


@pytest.mark.parametrize("d,vb", [(128, 2), (256, 2), (128, 4), (256, 4)])
def test_value_code_byte_order_is_a_permutation(lib, d, vb):
    cfg = _lib.tq_config(d, 3, vb, 32)
    row = d * vb // 8
    seen = np.zeros(16 * row, dtype=np.int32)
    for tok in range(16):
        for b in range(row):
            off = lib.tq_vcode_native_offset(C.byref(cfg), tok, b)
            assert 0 <= off < 16 * row
            seen[off] += 1
    assert (seen == 1).all()
    assert lib.tq_vcode_native_offset(C.byref(cfg), 16, 0) == -7
    assert lib.tq_vcode_native_offset(C.byref(cfg), 0, row) == -7


def test_unsupported_configs_are_refused(lib):
    lay = _lib.tq_layout()
    for cfg in [(64, 3, 2, 32), (128, 2, 2, 32), (128, 5, 2, 32), (128, 3, 3, 32), (128, 3, 2, 64)]:
        c = _lib.tq_config(*cfg)
        assert lib.tq_get_layout(C.byref(c), C.byref(lay)) == -4
    assert b"outside the compiled set" in lib.tq_strerror(-4)
    assert lib.tq_strerror(0) == b"ok"
    assert b"sm_100a" in lib.tq_version()


def test_workspace_sizes(lib):
    cfg = _lib.tq_config(256, 3, 2, 32)
    out = C.c_size_t(0)
    assert lib.tq_decode_workspace_bytes(C.byref(cfg), 1, 16, 4, 37, C.byref(out)) == 0
    assert out.value > 4 * 45 * 4 * 258 * 4
    assert lib.tq_decode_workspace_bytes(C.byref(cfg), 1, 15, 4, 37, C.byref(out)) == -4
    assert lib.tq_decode_workspace_bytes(C.byref(cfg), 0, 16, 4, 37, C.byref(out)) == -2
    assert lib.tq_scores_workspace_bytes(C.byref(cfg), 8, C.byref(out)) == 0
    assert out.value == 256 + 8 * 2 * 256 * 4


def test_null_and_shape_errors_come_before_any_launch(lib):
    consts = _lib.tq_consts()
    consts.cfg = _lib.tq_config(128, 3, 2, 32)
    pool = _lib.tq_pool(None, 4, 2)
    assert lib.tq_store(C.byref(consts), None, None, 1, 16, 2, 256, 128, None, None, 0, C.byref(pool), None) == -1
    args = _lib.tq_decode_args()
    assert lib.tq_decode(C.byref(consts), C.byref(pool), C.byref(args), None) == -1
    assert lib.tq_decode(None, None, None, None) == -1
    assert lib.tq_decode_host_io(C.byref(consts), C.byref(pool), None, None, None, 0, None, 0, None) == -1
    assert lib.tq_decode_host_io(C.byref(consts), C.byref(pool), C.byref(args), None, None, 0, None, 0, None) == -1
    assert lib.tq_decode_static(C.byref(consts), C.byref(pool), None, None) == -1
    assert lib.tq_scores(C.byref(consts), C.byref(pool), None, 16, None, 0, 1, None, None, 0, None) == -1
    assert lib.tq_workspace_init(None, 1024, None) == -1

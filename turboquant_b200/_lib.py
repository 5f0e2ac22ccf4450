"""ctypes binding of libturboquant_b200.so (declarations: include/turboquant_b200.h).

There is no CPU fallback: if the library is missing or a call fails, the
error is raised.
"""

from __future__ import annotations

import ctypes as C
import os

from .build import LIB_PATH

TQ_BLOCK_TOKENS = 16
TQ_MAX_CENTROIDS = 16
TQ_F32, TQ_BF16, TQ_F16 = 0, 1, 2
TQ_ERR_UNSUPPORTED = -4


class TQError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: {strerror(status)} (status {status})")


class tq_config(C.Structure):
    _fields_ = [("head_dim", C.c_int32), ("key_bits", C.c_int32), ("value_bits", C.c_int32),
                ("group_size", C.c_int32)]


class tq_consts(C.Structure):
    _fields_ = [("cfg", tq_config), ("pi", C.c_void_p), ("pi_t", C.c_void_p), ("s", C.c_void_p),
                ("s_t", C.c_void_p), ("centroids", C.c_float * TQ_MAX_CENTROIDS),
                ("boundaries", C.c_float * TQ_MAX_CENTROIDS), ("qjl_scale", C.c_float),
                ("pi_limbs", C.c_void_p * 3), ("m_limbs", C.c_void_p * 2), ("s_limbs", C.c_void_p * 2)]


class tq_layout(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "block_tokens", "kcode_row", "ksign_row", "vcode_row", "n_groups", "off_kcodes", "off_ksigns",
        "off_knorm", "off_krnorm", "off_vcodes", "off_vscale", "off_vzero", "block_bytes", "bytes_per_token")]


class tq_pool(C.Structure):
    _fields_ = [("base", C.c_void_p), ("num_blocks", C.c_int64), ("num_kv_heads", C.c_int32)]


class tq_planes(C.Structure):
    _fields_ = [("mse_indices", C.c_void_p), ("qjl_signs", C.c_void_p), ("norms", C.c_void_p),
                ("residual_norms", C.c_void_p), ("v_data", C.c_void_p), ("v_scales", C.c_void_p),
                ("v_zeros", C.c_void_p), ("capacity", C.c_int64)]


class tq_decode_args(C.Structure):
    _fields_ = [("query", C.c_void_p), ("q_dtype", C.c_int32), ("batch", C.c_int32), ("num_q_heads", C.c_int32),
                ("block_table", C.c_void_p), ("block_table_stride", C.c_int32), ("seq_lens", C.c_void_p),
                ("max_seq_len", C.c_int32), ("min_history", C.c_int32), ("ring_k", C.c_void_p),
                ("ring_v", C.c_void_p), ("ring_dtype", C.c_int32), ("ring_lens", C.c_void_p),
                ("max_ring_len", C.c_int32), ("ring_stride_seq", C.c_int64), ("ring_stride_token", C.c_int64),
                ("scale", C.c_float), ("out", C.c_void_p), ("workspace", C.c_void_p),
                ("workspace_bytes", C.c_size_t), ("num_splits", C.c_int32), ("query_prepared", C.c_int32), ("kernel", C.c_int32), ("append_k", C.c_void_p), ("append_v", C.c_void_p),
                ("ring_capacity", C.c_int32)]


# name -> (restype, argtypes); every symbol include/turboquant_b200.h declares
SIGNATURES = {
    "tq_get_layout": (C.c_int, [C.POINTER(tq_config), C.POINTER(tq_layout)]),
    "tq_vcode_native_offset": (C.c_int, [C.POINTER(tq_config), C.c_int32, C.c_int32]),
    "tq_decode_workspace_bytes": (C.c_int, [C.POINTER(tq_config), C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                            C.POINTER(C.c_size_t)]),
    "tq_scores_workspace_bytes": (C.c_int, [C.POINTER(tq_config), C.c_int64, C.POINTER(C.c_size_t)]),
    "tq_strerror": (C.c_char_p, [C.c_int]),
    "tq_version": (C.c_char_p, []),
    "tq_store": (C.c_int, [C.POINTER(tq_consts), C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int32,
                           C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.POINTER(tq_pool),
                           C.c_void_p]),
    "tq_store_paged": (C.c_int, [C.POINTER(tq_consts), C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int32, C.c_int32,
                                 C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
                                 C.POINTER(tq_pool), C.c_void_p]),
    "tq_store_read_status": (C.c_int, [C.POINTER(C.c_int32)]),
    "tq_prefill_attention": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int32,
                                       C.c_int32, C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                       C.c_int64, C.c_float, C.c_void_p]),
    "tq_prefill_attention_read_status": (C.c_int, [C.POINTER(C.c_int32)]),
    "tq_decode": (C.c_int, [C.POINTER(tq_consts), C.POINTER(tq_pool), C.POINTER(tq_decode_args), C.c_void_p]),
    "tq_decode_host_io": (C.c_int, [C.POINTER(tq_consts), C.POINTER(tq_pool), C.POINTER(tq_decode_args), C.c_void_p,
                                    C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p]),
    "tq_decode_static": (C.c_int, [C.POINTER(tq_consts), C.POINTER(tq_pool), C.POINTER(tq_decode_args), C.c_void_p]),
    "tq_decode_static_scratch_bytes": (C.c_size_t, []),
    "tq_decode_static_read_status": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32)]),
    "tq_host_buffer_forget": (C.c_int, [C.c_void_p]),
    "tq_scores": (C.c_int, [C.POINTER(tq_consts), C.POINTER(tq_pool), C.c_void_p, C.c_int64, C.c_void_p, C.c_int,
                            C.c_int32, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "tq_pool_to_planes": (C.c_int, [C.POINTER(tq_config), C.POINTER(tq_pool), C.c_void_p, C.c_int64,
                                    C.POINTER(tq_planes), C.c_void_p]),
    "tq_planes_to_pool": (C.c_int, [C.POINTER(tq_config), C.POINTER(tq_planes), C.c_int64, C.c_void_p, C.c_int64,
                                    C.POINTER(tq_pool), C.c_void_p]),
    "tq_dequant_keys": (C.c_int, [C.POINTER(tq_consts), C.POINTER(tq_pool), C.c_void_p, C.c_int64, C.c_int32,
                                  C.c_void_p, C.c_void_p]),
    "tq_dequant_values": (C.c_int, [C.POINTER(tq_config), C.POINTER(tq_pool), C.c_void_p, C.c_int64, C.c_void_p,
                                    C.c_void_p]),
    "tq_pack_stage": (C.c_int, [C.POINTER(tq_consts), C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p,
                                C.c_void_p]),
    "tq_workspace_init": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p]),
    "tq_read_status": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_int32)]),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        path = LIB_PATH
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: build it with `python -m turboquant_b200.build` "
                "(there is no CPU or PyTorch fallback for this path)")
        handle = C.CDLL(path)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def strerror(status: int) -> str:
    return lib().tq_strerror(status).decode()


def check(status: int, where: str) -> None:
    if status != 0:
        raise TQError(status, where)

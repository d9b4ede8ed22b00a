"""ctypes binding of the C-ABI in include/b200q.h.

Loading fails loudly when libb200q.so has not been built; there is no Python or
CPU fallback for any compute entry point.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
# B200Q_LIB selects another build of the same library (the trace build, `python -m brotensor_b200.build --trace`)
LIB_PATH = os.environ.get("B200Q_LIB") or os.path.join(PKG, "lib", "libb200q.so")

OK = 0
ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_TIMEOUT, ERR_WORKSPACE = 1, 2, 3, 4, 5
Q8_0, Q4_K, Q6_K = 14, 22, 24
Q4_0, Q5_K = 10, 23  # carried by brotensor's loader without ops; decode, GEMV (plain-load kernel) and gather here
Q6_K_R8 = 124  # Q6_K regrouped by field in runs of eight blocks (b200q_repack)
F32, F16, BF16 = 0, 1, 4

# Every symbol include/b200q.h declares: (name, restype, argtypes)
_vp, _i, _sz, _i64 = C.c_void_p, C.c_int, C.c_size_t, C.c_int64
SYMBOLS = [
    ("b200q_abi_version", _i, []),
    ("b200q_status_str", C.c_char_p, [_i]),
    ("b200q_last_error", C.c_char_p, []),
    ("b200q_block_elems", _i, [_i]),
    ("b200q_block_bytes", _i, [_i]),
    ("b200q_packed_bytes", _sz, [_i, _i64, _i]),
    ("b200q_repacked_fmt", _i, [_i, _i]),
    ("b200q_repack", _i, [_i, _vp, _vp, _i64, _i, _vp]),
    ("b200q_unpack", _i, [_i, _vp, _vp, _i64, _i, _vp]),
    ("b200q_dequant", _i, [_i, _vp, _vp, _i, _i64, _i, _vp]),
    ("b200q_embedding_gather", _i, [_i, _vp, _vp, _i, _i64, _i, _vp, _i, _vp]),
    ("b200q_gemv", _i, [_i, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp]),
    ("b200q_gemv_multi_rmsnorm", _i, [_i, _i, C.POINTER(_vp), C.POINTER(_i), C.POINTER(_vp), C.POINTER(_vp), _vp, _i, _vp, C.c_float, _i, _i, _vp]),
    ("b200q_gemv_swiglu", _i, [_i, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _vp]),
    ("b200q_gemv_multi", _i, [_i, _i, C.POINTER(_vp), C.POINTER(_i), C.POINTER(_vp), C.POINTER(_vp), _vp, _i, _i, _i, _vp]),
    ("b200q_gemv_shard", _i, [_i, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, C.POINTER(_vp), _vp, _vp]),
    ("b200q_gemv_shard_topk", _i, [_i, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, C.POINTER(_vp), C.POINTER(_vp), _vp, _i, _vp, _vp, _vp]),
    ("b200q_gemm_workspace_bytes", _sz, [_i, _i, _i, _i, _i]),
    ("b200q_gemm", _i, [_i, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp, _sz, _vp]),
    ("b200q_gemm_static_max_bytes", _sz, []),
    ("b200q_gemm_static", _i, [_i, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp]),
    ("b200q_linear", _i, [_i, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp, _sz, _vp]),
    ("b200q_tc_calls_consume", C.c_ulonglong, [_i]),
    ("brotensor_q4k_wmma_calls_consume", C.c_ulonglong, []),
    ("brotensor_q6k_wmma_calls_consume", C.c_ulonglong, []),
    ("brotensor_q8_0_wmma_calls_consume", C.c_ulonglong, []),
    ("b200q_device_status", _i, [C.POINTER(_i)]),
    ("b200q_set_option", _i, [C.c_char_p, _i]),
    ("b200q_get_option", _i, [C.c_char_p, C.POINTER(_i)]),
]


class B200QError(RuntimeError):
    def __init__(self, status: int, msg: str):
        super().__init__(f"b200q: {msg} (status {status})")
        self.status = status


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m brotensor_b200.build` "
                "(nvcc, sm_100a). There is no fallback path.")
        L = C.CDLL(LIB_PATH)
        for name, res, args in SYMBOLS:
            f = getattr(L, name)
            f.restype = res
            f.argtypes = args
        _lib = L
    return _lib


def check(status: int) -> None:
    if status != OK:
        raise B200QError(status, lib().b200q_last_error().decode() or lib().b200q_status_str(status).decode())

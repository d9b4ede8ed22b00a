"""ctypes binding of the flat C entry points of the C++ host layer
(brotensor_b200/host/c_api.cpp): weights as Tensor handles, sessions that run one
linear layer from host activations to host results through Tensor / dispatch / the
public ops. Used by the benchmark's end-to-end arm and by tests."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "lib", "libbrotensor_b200.so")
_NP = {0: np.float32, 1: np.float16, 4: np.uint16}  # bf16 travels as raw 16-bit patterns

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m brotensor_b200.build`")
        L = C.CDLL(LIB_PATH)
        L.b200h_last_error.restype = C.c_char_p
        L.b200h_weight_from_host.restype = C.c_void_p
        L.b200h_weight_from_host.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int]
        L.b200h_tensor_free.argtypes = [C.c_void_p]
        L.b200h_tensor_data.restype = C.c_void_p
        L.b200h_tensor_data.argtypes = [C.c_void_p]
        L.b200h_dequant.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.b200h_session_create.restype = C.c_void_p
        L.b200h_session_create.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
        L.b200h_session_free.argtypes = [C.c_void_p]
        L.b200h_session_run.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        _lib = L
    return _lib


def _check(ok: bool):
    if not ok:
        raise RuntimeError(lib().b200h_last_error().decode())


def init() -> int:
    n = lib().b200h_init()
    _check(n >= 0)
    return n


class Weight:
    def __init__(self, fmt: int, blocks: np.ndarray, rows: int, cols: int, device: int = 0):
        blocks = np.ascontiguousarray(blocks, np.uint8)
        self.h = lib().b200h_weight_from_host(fmt, blocks.ctypes.data, rows, cols, device)
        _check(bool(self.h))
        self.fmt, self.rows, self.cols = fmt, rows, cols

    def dequant(self, out_dtype: int = 1) -> np.ndarray:
        out = np.empty((self.rows, self.cols), _NP[out_dtype])
        _check(lib().b200h_dequant(self.h, out.ctypes.data, out_dtype) == 0)
        return out

    def close(self):
        if self.h:
            lib().b200h_tensor_free(self.h)
            self.h = None


class Session:
    """One linear layer: run(x_host) -> y_host, copies included."""

    def __init__(self, W: Weight, M: int, x_dtype: int = 0, y_dtype: int = 0, bias: np.ndarray | None = None):
        self.W, self.M = W, M
        self.y = np.empty((M, W.rows), _NP[y_dtype])
        b = None if bias is None else np.ascontiguousarray(bias)
        self.h = lib().b200h_session_create(W.h, M, x_dtype, y_dtype, None if b is None else b.ctypes.data)
        _check(bool(self.h))

    def run(self, x: np.ndarray) -> np.ndarray:
        _check(lib().b200h_session_run(self.h, x.ctypes.data, self.y.ctypes.data) == 0)
        return self.y

    def close(self):
        if self.h:
            lib().b200h_session_free(self.h)
            self.h = None

"""ctypes front end of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Only tests/, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline and
reference arms may import this package; the product library never does.

``cpu``  -> liboracle.so : plain-C restatement (oracle/b200q_oracle.c)
``ref``  -> _ref/libref.so : brotensor's own host reference, compiled from the
            reference tree by oracle/Makefile (None when it was never built).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
Q8_0, Q4_K, Q6_K = 14, 22, 24
Q4_0, Q5_K = 10, 23  # decoders restated from the ggml block definitions (the reference has none)
BLOCK_ELEMS = {Q8_0: 32, Q4_K: 256, Q6_K: 256, Q4_0: 32, Q5_K: 256}
BLOCK_BYTES = {Q8_0: 34, Q4_K: 144, Q6_K: 210, Q4_0: 18, Q5_K: 176}

_u8p = C.POINTER(C.c_uint8)
_f32p = C.POINTER(C.c_float)
_f64p = C.POINTER(C.c_double)
_u16p = C.POINTER(C.c_uint16)


# where the reference checkout lives when it is available (the Makefile's REF)
REF_TREE = os.environ.get("BROTENSOR_REF", os.path.join(os.sep, "root", "reference"))


def build(force: bool = False) -> None:
    """Compile liboracle.so (and _ref/libref.so where the reference tree exists)."""
    if force or not os.path.exists(os.path.join(HERE, "liboracle.so")) or (
        os.path.isdir(os.path.join(REF_TREE, "tests")) and not os.path.exists(os.path.join(HERE, "_ref", "libref.so"))
    ):
        subprocess.run(["make", "-s", "-C", HERE, "REF=" + REF_TREE], check=True)


def build_gpu() -> None:
    """GPU-side checker builds (cross-compiled; see the Makefile's `gpu` target): brotensor's core with its
    own CUDA quant kernels (_ref/libref_cuda.so, the same-box comparator) and brotensor's own parity tests
    linked against this repository's binding (_ref/b200_test_*). Needs the reference tree and a built
    libb200q.so; a no-op where the tree is absent (the prebuilt files travel)."""
    if os.path.isdir(os.path.join(REF_TREE, "tests")):
        subprocess.run(["make", "-s", "-C", HERE, "gpu", "REF=" + REF_TREE, "-j8"], check=True)


def _ptr(a: np.ndarray, t):
    return a.ctypes.data_as(t)


class _Cpu:
    def __init__(self) -> None:
        build()
        L = self.lib = C.CDLL(os.path.join(HERE, "liboracle.so"))
        L.oracle_fp16_to_fp32.restype = C.c_float
        L.oracle_fp16_to_fp32.argtypes = [C.c_uint16]
        L.oracle_fp32_to_fp16.restype = C.c_uint16
        L.oracle_fp32_to_fp16.argtypes = [C.c_float]
        L.oracle_bf16_to_fp32.restype = C.c_float
        L.oracle_bf16_to_fp32.argtypes = [C.c_uint16]
        L.oracle_fp32_to_bf16.restype = C.c_uint16
        L.oracle_fp32_to_bf16.argtypes = [C.c_float]
        L.oracle_dequant_f32.argtypes = [C.c_int, _u8p, C.c_int64, C.c_int, _f32p]
        L.oracle_dequant_16.argtypes = [C.c_int, _u8p, C.c_int64, C.c_int, C.c_int, _u16p]
        L.oracle_matmul.argtypes = [C.c_int, _u8p, _f32p, _f32p, _f32p, _f64p] + [C.c_int] * 4
        L.oracle_q4k_unpack_sc_m.argtypes = [_u8p, _u8p, _u8p]
        L.oracle_q4k_pack_sc_m.argtypes = [_u8p, _u8p, _u8p]

    def dequant_f32(self, fmt: int, W: np.ndarray, rows: int, K: int) -> np.ndarray:
        W = np.ascontiguousarray(W, dtype=np.uint8)
        assert W.size == rows * (K // BLOCK_ELEMS[fmt]) * BLOCK_BYTES[fmt]
        out = np.empty((rows, K), np.float32)
        assert self.lib.oracle_dequant_f32(fmt, _ptr(W, _u8p), rows, K, _ptr(out, _f32p)) == 0
        return out

    def dequant_16(self, fmt: int, W: np.ndarray, rows: int, K: int, kind: int) -> np.ndarray:
        """kind 1 = fp16 bits, 4 = bf16 bits (round to nearest even of the fp32 decode)."""
        W = np.ascontiguousarray(W, dtype=np.uint8)
        out = np.empty((rows, K), np.uint16)
        assert self.lib.oracle_dequant_16(fmt, _ptr(W, _u8p), rows, K, kind, _ptr(out, _u16p)) == 0
        return out

    def matmul(self, fmt, W, X, bias=None, threads=1, want_f64=False):
        """Y(M,N) = X(M,K) @ decode(W(N,K)).T (+bias); sequential fp32 dot per output."""
        W = np.ascontiguousarray(W, dtype=np.uint8)
        X = np.ascontiguousarray(X, dtype=np.float32)
        M, K = X.shape
        N = W.size // ((K // BLOCK_ELEMS[fmt]) * BLOCK_BYTES[fmt])
        Y = np.empty((M, N), np.float32)
        Y64 = np.empty((M, N), np.float64) if want_f64 else None
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32).reshape(-1)
        rc = self.lib.oracle_matmul(fmt, _ptr(W, _u8p), _ptr(X, _f32p), None if b is None else _ptr(b, _f32p),
                                    _ptr(Y, _f32p), None if Y64 is None else _ptr(Y64, _f64p), M, N, K, threads)
        assert rc == 0
        return (Y, Y64) if want_f64 else Y

    def q4k_unpack_sc_m(self, s12: np.ndarray):
        s12 = np.ascontiguousarray(s12, np.uint8)
        sc = np.empty(8, np.uint8)
        m = np.empty(8, np.uint8)
        self.lib.oracle_q4k_unpack_sc_m(_ptr(s12, _u8p), _ptr(sc, _u8p), _ptr(m, _u8p))
        return sc, m

    def q4k_pack_sc_m(self, sc, m):
        sc = np.ascontiguousarray(sc, np.uint8)
        m = np.ascontiguousarray(m, np.uint8)
        s = np.empty(12, np.uint8)
        self.lib.oracle_q4k_pack_sc_m(_ptr(s, _u8p), _ptr(sc, _u8p), _ptr(m, _u8p))
        return s

    def fp16_to_fp32(self, bits):
        return np.array([self.lib.oracle_fp16_to_fp32(int(b)) for b in np.asarray(bits).ravel()], np.float32)

    def fp32_to_fp16(self, v):
        return np.array([self.lib.oracle_fp32_to_fp16(float(x)) for x in np.asarray(v, np.float32).ravel()], np.uint16)

    def fp32_to_bf16(self, v):
        return np.array([self.lib.oracle_fp32_to_bf16(float(x)) for x in np.asarray(v, np.float32).ravel()], np.uint16)


class _Ref:
    def __init__(self, path: str) -> None:
        L = self.lib = C.CDLL(path)
        L.ref_rng_seed.argtypes = [C.c_uint32]
        L.ref_rng_uniform.argtypes = [C.c_float, C.c_float, C.c_int64, _f32p]
        L.ref_fp32_to_fp16_bits.restype = C.c_uint16
        L.ref_fp32_to_fp16_bits.argtypes = [C.c_float]
        L.ref_fp16_bits_to_fp32.restype = C.c_float
        L.ref_fp16_bits_to_fp32.argtypes = [C.c_uint16]
        L.ref_fp32_to_bf16_bits.restype = C.c_uint16
        L.ref_fp32_to_bf16_bits.argtypes = [C.c_float]
        L.ref_quantize_rows.argtypes = [C.c_int, _f32p, C.c_int64, C.c_int, _u8p]
        L.ref_dequant_rows.argtypes = [C.c_int, _u8p, C.c_int64, C.c_int, _f32p]
        L.ref_matmul.argtypes = [C.c_int, _u8p, _f32p, _f32p, _f32p] + [C.c_int] * 4
        L.ref_q4k_pack_sc_m.argtypes = [_u8p, _u8p, _u8p]
        L.ref_q4k_unpack_sc_m.argtypes = [_u8p, _u8p, _u8p]
        L.ref_gguf_open.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
        L.ref_shape_to_2d.argtypes = [C.POINTER(C.c_int64), C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int),
                                      C.c_char_p, C.c_int]

    def seed(self, s: int) -> None:
        self.lib.ref_rng_seed(s)

    def uniform(self, lo: float, hi: float, n: int) -> np.ndarray:
        out = np.empty(n, np.float32)
        self.lib.ref_rng_uniform(lo, hi, n, _ptr(out, _f32p))
        return out

    def quantize(self, fmt: int, Wf: np.ndarray) -> np.ndarray:
        Wf = np.ascontiguousarray(Wf, np.float32)
        rows, K = Wf.shape
        out = np.zeros(rows * (K // BLOCK_ELEMS[fmt]) * BLOCK_BYTES[fmt], np.uint8)
        assert self.lib.ref_quantize_rows(fmt, _ptr(Wf, _f32p), rows, K, _ptr(out, _u8p)) == 0
        return out

    def dequant_f32(self, fmt: int, W: np.ndarray, rows: int, K: int) -> np.ndarray:
        W = np.ascontiguousarray(W, np.uint8)
        out = np.empty((rows, K), np.float32)
        assert self.lib.ref_dequant_rows(fmt, _ptr(W, _u8p), rows, K, _ptr(out, _f32p)) == 0
        return out

    def matmul(self, fmt, W, X, bias=None, threads=1):
        W = np.ascontiguousarray(W, np.uint8)
        X = np.ascontiguousarray(X, np.float32)
        M, K = X.shape
        N = W.size // ((K // BLOCK_ELEMS[fmt]) * BLOCK_BYTES[fmt])
        Y = np.empty((M, N), np.float32)
        b = None if bias is None else np.ascontiguousarray(bias, np.float32).reshape(-1)
        assert self.lib.ref_matmul(fmt, _ptr(W, _u8p), _ptr(X, _f32p), None if b is None else _ptr(b, _f32p),
                                   _ptr(Y, _f32p), M, N, K, threads) == 0
        return Y

    def fp32_to_fp16(self, v):
        return np.array([self.lib.ref_fp32_to_fp16_bits(float(x)) for x in np.asarray(v, np.float32).ravel()], np.uint16)

    def fp16_to_fp32(self, bits):
        return np.array([self.lib.ref_fp16_bits_to_fp32(int(b)) for b in np.asarray(bits).ravel()], np.float32)

    def fp32_to_bf16(self, v):
        return np.array([self.lib.ref_fp32_to_bf16_bits(float(x)) for x in np.asarray(v, np.float32).ravel()], np.uint16)


_cpu = None
_ref = None


def cpu() -> _Cpu:
    global _cpu
    if _cpu is None:
        _cpu = _Cpu()
    return _cpu


def ref():
    """brotensor's own host reference, or None when oracle/_ref was never built."""
    global _ref
    if _ref is None:
        p = os.path.join(HERE, "_ref", "libref.so")
        if not os.path.exists(p):
            if os.path.isdir(os.path.join(REF_TREE, "tests")):
                build(force=True)
            else:
                return None
        _ref = _Ref(p)
    return _ref


def rel_l2(got: np.ndarray, want: np.ndarray) -> float:
    g = np.asarray(got, np.float64).ravel()
    w = np.asarray(want, np.float64).ravel()
    den = float(np.sqrt(np.sum(w * w)))
    return float(np.sqrt(np.sum((g - w) ** 2))) / (den if den > 0 else 1.0)

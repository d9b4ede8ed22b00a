"""Thin torch-tensor front end of the C-ABI, used by the tests and the benchmark.

Argument meaning follows brotensor's ops (include/brotensor/ops/quant.h): W is a
(N, K) quantized weight given as its raw GGUF block bytes, X is (M, K), the
result is (M, N). torch only supplies device memory and the current stream.
"""
from __future__ import annotations

import torch

from . import _capi as capi
from .synth import BLOCK_BYTES, BLOCK_ELEMS

_DT = {torch.float32: capi.F32, torch.float16: capi.F16, torch.bfloat16: capi.BF16}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check_w(fmt: int, W: torch.Tensor, N: int, K: int) -> None:
    if W.dtype != torch.uint8 or not W.is_cuda or not W.is_contiguous():
        raise ValueError("W must be a contiguous CUDA uint8 tensor holding raw GGUF blocks")
    if K % BLOCK_ELEMS[fmt]:
        raise ValueError(f"K ({K}) must be a multiple of {BLOCK_ELEMS[fmt]}")
    need = N * (K // BLOCK_ELEMS[fmt]) * BLOCK_BYTES[fmt]
    if W.numel() != need:
        raise ValueError(f"W holds {W.numel()} bytes, ({N}, {K}) needs {need}")


def repacked_fmt(fmt: int, K: int) -> int:
    """Format code of the device-side repacked form of raw format `fmt` for rows of K elements (`fmt` itself: none)."""
    return capi.lib().b200q_repacked_fmt(fmt, K)


def repack(fmt: int, W: torch.Tensor, N: int, K: int, inplace: bool = False) -> torch.Tensor:
    """Raw GGUF rows -> the layout the kernels read fastest (same size, bit-identical content)."""
    _check_w(fmt, W, N, K)
    out = W if inplace else torch.empty_like(W)
    with torch.cuda.device(W.device):
        capi.check(capi.lib().b200q_repack(fmt, W.data_ptr(), out.data_ptr(), N, K, _stream()))
    return out


def unpack(fmt: int, W: torch.Tensor, N: int, K: int, inplace: bool = False) -> torch.Tensor:
    """Inverse of repack; `fmt` is the raw format."""
    _check_w(fmt, W, N, K)
    out = W if inplace else torch.empty_like(W)
    with torch.cuda.device(W.device):
        capi.check(capi.lib().b200q_unpack(fmt, W.data_ptr(), out.data_ptr(), N, K, _stream()))
    return out


def dequant(fmt: int, W: torch.Tensor, N: int, K: int, out_dtype=torch.float16) -> torch.Tensor:
    _check_w(fmt, W, N, K)
    out = torch.empty((N, K), dtype=out_dtype, device=W.device)
    with torch.cuda.device(W.device):
        capi.check(capi.lib().b200q_dequant(fmt, W.data_ptr(), out.data_ptr(), _DT[out_dtype], N, K, _stream()))
    return out


def embedding_gather(fmt: int, table: torch.Tensor, idx: torch.Tensor, rows: int, K: int, out_dtype=torch.float16) -> torch.Tensor:
    """out[b] = decode(table row idx[b]); idx: int32 device tensor. Rows outside the table come back as zeros."""
    _check_w(fmt, table, rows, K)
    if idx.dtype != torch.int32 or not idx.is_cuda or not idx.is_contiguous():
        raise ValueError("idx must be a contiguous CUDA int32 tensor")
    B = idx.numel()
    out = torch.empty((B, K), dtype=out_dtype, device=table.device)
    with torch.cuda.device(table.device):
        capi.check(capi.lib().b200q_embedding_gather(fmt, table.data_ptr(), idx.data_ptr(), B, rows, K, out.data_ptr(), _DT[out_dtype], _stream()))
    return out


def _linear(entry: str, fmt, W, X, N, bias, out, out_dtype, ws):
    if X.dim() == 1:
        X = X.unsqueeze(0)
    M, K = X.shape
    _check_w(fmt, W, N, K)
    if not X.is_contiguous():
        raise ValueError("X must be contiguous")
    if bias is not None and (bias.dtype != X.dtype or bias.numel() != N):
        raise ValueError("bias must have N elements of X's dtype")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or (torch.float16 if X.dtype == torch.float16 else torch.float32),
                          device=X.device)
    L = capi.lib()
    bptr = bias.data_ptr() if bias is not None else None
    with torch.cuda.device(W.device):
        if entry in ("gemv", "gemm_static"):
            f = L.b200q_gemv if entry == "gemv" else L.b200q_gemm_static
            rc = f(fmt, W.data_ptr(), X.data_ptr(), _DT[X.dtype], bptr, out.data_ptr(), _DT[out.dtype],
                              M, N, K, _stream())
        else:
            need = L.b200q_gemm_workspace_bytes(fmt, _DT[X.dtype], M, N, K)
            if ws is None and need:
                ws = torch.empty(need, dtype=torch.uint8, device=X.device)
            f = L.b200q_gemm if entry == "gemm" else L.b200q_linear
            rc = f(fmt, W.data_ptr(), X.data_ptr(), _DT[X.dtype], bptr, out.data_ptr(), _DT[out.dtype], M, N, K,
                   ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0, _stream())
    capi.check(rc)
    return out


def gemv(fmt, W, X, N, bias=None, out=None, out_dtype=None):
    """Y(M,N) = X(M,K) @ decode(W).T (+bias), 1 <= M <= 8."""
    return _linear("gemv", fmt, W, X, N, bias, out, out_dtype, None)


def gemv_swiglu(fmt, W_gate, W_up, x, N, out=None, out_dtype=None):
    """y(1, N) = silu(x @ decode(W_gate).T) * (x @ decode(W_up).T) in one launch."""
    x = x.reshape(1, -1)
    K = x.shape[1]
    _check_w(fmt, W_gate, N, K)
    _check_w(fmt, W_up, N, K)
    if out is None:
        out = torch.empty((1, N), dtype=out_dtype or (torch.float16 if x.dtype == torch.float16 else torch.float32), device=x.device)
    with torch.cuda.device(x.device):
        capi.check(capi.lib().b200q_gemv_swiglu(fmt, W_gate.data_ptr(), W_up.data_ptr(), x.data_ptr(), _DT[x.dtype],
                                               out.data_ptr(), _DT[out.dtype], N, K, _stream()))
    return out


def gemv_multi(fmt, Ws, x, Ns, outs=None, biases=None):
    """Several matrices against one activation vector in one launch; returns the list of (1, N_s) results."""
    import ctypes as C
    n = len(Ws)
    K = x.numel()
    for W, N in zip(Ws, Ns):
        _check_w(fmt, W, N, K)
    if outs is None:
        outs = [torch.empty((1, N), dtype=torch.float32, device=x.device) for N in Ns]
    Wp = (C.c_void_p * n)(*[W.data_ptr() for W in Ws])
    Yp = (C.c_void_p * n)(*[y.data_ptr() for y in outs])
    Np = (C.c_int * n)(*Ns)
    Bp = None if biases is None else (C.c_void_p * n)(*[(b.data_ptr() if b is not None else None) for b in biases])
    with torch.cuda.device(x.device):
        rc = capi.lib().b200q_gemv_multi(fmt, n, Wp, Np, Yp, Bp, x.data_ptr(), _DT[x.dtype], _DT[outs[0].dtype], K, _stream())
    capi.check(rc)
    return outs


def gemv_multi_rmsnorm(fmt, Ws, x, gamma, eps, Ns, outs=None):
    """gemv_multi on rms_norm(x) * gamma, the normalisation folded into the kernel."""
    import ctypes as C
    n = len(Ws)
    K = x.numel()
    for W, N in zip(Ws, Ns):
        _check_w(fmt, W, N, K)
    if gamma.dtype != x.dtype or gamma.numel() != K:
        raise ValueError("gamma must have K elements of x's dtype")
    if outs is None:
        outs = [torch.empty((1, N), dtype=torch.float32, device=x.device) for N in Ns]
    Wp = (C.c_void_p * n)(*[W.data_ptr() for W in Ws])
    Yp = (C.c_void_p * n)(*[y.data_ptr() for y in outs])
    Np = (C.c_int * n)(*Ns)
    with torch.cuda.device(x.device):
        rc = capi.lib().b200q_gemv_multi_rmsnorm(fmt, n, Wp, Np, Yp, None, x.data_ptr(), _DT[x.dtype], gamma.data_ptr(), float(eps),
                                                 _DT[outs[0].dtype], K, _stream())
    capi.check(rc)
    return outs


def gemm(fmt, W, X, N, bias=None, out=None, out_dtype=None, ws=None):
    """Prefill GEMM on the tensor cores, any M."""
    return _linear("gemm", fmt, W, X, N, bias, out, out_dtype, ws)


def gemm_static(fmt, W, X, N, bias=None, out=None, out_dtype=None):
    """The GEMM with its scratch in the library's fixed device array: makes no allocation."""
    return _linear("gemm_static", fmt, W, X, N, bias, out, out_dtype, None)


def linear(fmt, W, X, N, bias=None, out=None, out_dtype=None, ws=None):
    """Routing of the batched ops: M <= 8 -> gemv, else gemm."""
    return _linear("linear", fmt, W, X, N, bias, out, out_dtype, ws)


def set_option(key: str, value: int) -> None:
    capi.check(capi.lib().b200q_set_option(key.encode(), value))


def device_status() -> int:
    """Synchronises; returns 0 or raises if a kernel's bounded wait ran out."""
    import ctypes
    v = ctypes.c_int(0)
    capi.check(capi.lib().b200q_device_status(ctypes.byref(v)))
    return v.value


def tc_calls_consume(fmt: int) -> int:
    return int(capi.lib().b200q_tc_calls_consume(fmt))

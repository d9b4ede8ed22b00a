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
        L.b200h_weight_view.restype = C.c_void_p
        L.b200h_weight_view.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int]
        L.b200h_weight_repack.argtypes = [C.c_void_p]
        L.b200h_weight_unpack.argtypes = [C.c_void_p]
        L.b200h_weight_is_repacked.argtypes = [C.c_void_p]
        L.b200h_tensor_to_host.argtypes = [C.c_void_p, C.c_void_p]
        L.b200h_tensor_data.restype = C.c_void_p
        L.b200h_tensor_data.argtypes = [C.c_void_p]
        L.b200h_dequant.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.b200h_session_create.restype = C.c_void_p
        L.b200h_session_create.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
        L.b200h_session_free.argtypes = [C.c_void_p]
        L.b200h_session_run.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        L.b200h_session_enqueue.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        L.b200h_sync.argtypes = [C.c_int]
        L.b200h_layer_create.restype = C.c_void_p
        L.b200h_layer_create.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int]
        L.b200h_layer_free.argtypes = [C.c_void_p]
        L.b200h_layer_layout.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        L.b200h_layer_enqueue.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        L.b200h_capture_begin.restype = C.c_void_p
        L.b200h_capture_finish.restype = C.c_void_p
        L.b200h_capture_finish.argtypes = [C.c_void_p]
        L.b200h_graph_launch.argtypes = [C.c_void_p]
        L.b200h_graph_free.argtypes = [C.c_void_p]
        L.b200h_head_create.restype = C.c_void_p
        L.b200h_head_create.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
        L.b200h_head_connect.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.b200h_head_run.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        L.b200h_head_run_topk.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
        L.b200h_head_top_to_host.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        L.b200h_head_top_rows.restype = C.c_void_p
        L.b200h_head_top_rows.argtypes = [C.c_void_p]
        L.b200h_head_logits.restype = C.c_void_p
        L.b200h_head_logits.argtypes = [C.c_void_p]
        L.b200h_head_calls.restype = C.c_ulonglong
        L.b200h_head_calls.argtypes = [C.c_void_p]
        L.b200h_head_free.argtypes = [C.c_void_p]
        L.b200h_head_logits_to_host.argtypes = [C.c_void_p, C.c_void_p]
        L.b200h_set_stream.argtypes = [C.c_void_p, C.c_int]
        L.b200h_set_stream.restype = None
        _lib = L
    return _lib


def _check(ok: bool):
    if not ok:
        raise RuntimeError(lib().b200h_last_error().decode())


def init() -> int:
    n = lib().b200h_init()
    _check(n >= 0)
    return n


def set_stream(stream_ptr: int, device: int = -1) -> None:
    """Makes `stream_ptr` (a cudaStream_t as an int, 0 = legacy default) the calling thread's stream."""
    lib().b200h_set_stream(stream_ptr, device)


class Weight:
    def __init__(self, fmt: int, blocks: np.ndarray, rows: int, cols: int, device: int = 0):
        blocks = np.ascontiguousarray(blocks, np.uint8)
        self.h = lib().b200h_weight_from_host(fmt, blocks.ctypes.data, rows, cols, device)
        _check(bool(self.h))
        self.fmt, self.rows, self.cols = fmt, rows, cols

    @classmethod
    def view(cls, fmt: int, dev_ptr: int, rows: int, cols: int, device: int = 0) -> "Weight":
        """A Tensor of the host layer over quantized blocks that already live on the device
        (the caller keeps them alive)."""
        self = cls.__new__(cls)
        self.h = lib().b200h_weight_view(fmt, dev_ptr, rows, cols, device)
        _check(bool(self.h))
        self.fmt, self.rows, self.cols = fmt, rows, cols
        return self

    def repack(self) -> bool:
        """brotensor_b200::repack_weights: regroup the device bytes in place for aligned loads
        (bit-identical content). True when the weight is in that layout afterwards."""
        r = lib().b200h_weight_repack(self.h)
        _check(r >= 0)
        return bool(r)

    def unpack(self) -> None:
        _check(lib().b200h_weight_unpack(self.h) == 0)

    @property
    def repacked(self) -> bool:
        return bool(lib().b200h_weight_is_repacked(self.h))

    def raw_bytes(self) -> np.ndarray:
        """The tensor's device bytes as they are stored."""
        from .synth import packed_bytes
        out = np.empty(packed_bytes(self.fmt, self.rows, self.cols), np.uint8)
        _check(lib().b200h_tensor_to_host(self.h, out.ctypes.data) == 0)
        return out

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

    def enqueue(self, x_pinned_ptr: int, y_pinned_ptr: int) -> None:
        """Copy in, op, copy out enqueued on the calling thread's stream; page-locked host
        pointers; valid after sync(device)."""
        _check(lib().b200h_session_enqueue(self.h, x_pinned_ptr, y_pinned_ptr) == 0)

    def close(self):
        if self.h:
            lib().b200h_session_free(self.h)
            self.h = None


class LayerSet:
    """GEMV layers (M = 1) whose activations and results share one device arena each: a step is
    one copy in, the ops through the public signatures, one copy out. `x_off` / `y_off` are the
    byte offsets of every op's vector inside the arenas; host arenas use the same layout."""

    def __init__(self, weights, x_dtype: int = 0, y_dtype: int = 0):
        n = len(weights)
        arr = (C.c_void_p * n)(*[w.h for w in weights])
        self.h = lib().b200h_layer_create(arr, n, x_dtype, y_dtype)
        _check(bool(self.h))
        self.weights = list(weights)
        xo, yo = (C.c_ulonglong * n)(), (C.c_ulonglong * n)()
        xb, yb = C.c_ulonglong(), C.c_ulonglong()
        lib().b200h_layer_layout(self.h, xo, yo, C.byref(xb), C.byref(yb))
        self.x_off, self.y_off, self.x_bytes, self.y_bytes = list(xo), list(yo), xb.value, yb.value

    def enqueue(self, x_pinned_ptr: int, y_pinned_ptr: int) -> None:
        _check(lib().b200h_layer_enqueue(self.h, x_pinned_ptr, y_pinned_ptr) == 0)

    def close(self):
        if self.h:
            lib().b200h_layer_free(self.h)
            self.h = None


def sync(device: int = 0) -> None:
    _check(lib().b200h_sync(device) == 0)


class Graph:
    """brotensor_b200::CudaGraph: `with Graph.capture() as g: ...enqueue ops...` then g.launch()."""

    def __init__(self):
        self.h = None
        self._cap = None

    @classmethod
    def capture(cls) -> "Graph":
        return cls()

    def __enter__(self):
        self._cap = lib().b200h_capture_begin()
        _check(bool(self._cap))
        return self

    def __exit__(self, et, ev, tb):
        cap, self._cap = self._cap, None
        self.h = lib().b200h_capture_finish(cap)
        if et is None:
            _check(bool(self.h))
        return False

    def launch(self) -> None:
        _check(lib().b200h_graph_launch(self.h) == 0)

    def close(self):
        if self.h:
            lib().b200h_graph_free(self.h)
            self.h = None


class ShardedHead:
    """One rank of the row-sharded LM head (brotensor_b200::ShardedHead). `exchange` moves the
    64-byte IPC handles between the ranks: a callable taking this rank's handle (bytes) and
    returning all ranks' handles in rank order; None for a single rank."""

    def __init__(self, weight: "Weight", row_offset: int, total_rows: int, rank: int, world: int, exchange=None):
        hb = (C.c_ubyte * 64)()
        self.h = lib().b200h_head_create(weight.h, row_offset, total_rows, rank, world, hb)
        _check(bool(self.h))
        self.weight, self.total_rows, self.rank, self.world = weight, total_rows, rank, world
        if world > 1:
            allh = exchange(bytes(hb))
            assert len(allh) == world and all(len(x) == 64 for x in allh)
            buf = (C.c_ubyte * (64 * world)).from_buffer_copy(b"".join(allh))
            _check(lib().b200h_head_connect(self.h, buf, world) == 0)

    def run(self, x_dev_ptr: int, in_features: int, x_dtype: int = 0, weight: "Weight | None" = None) -> None:
        """Enqueues one forward; `weight` substitutes another tensor of the shard's shape."""
        _check(lib().b200h_head_run(self.h, weight.h if weight is not None else None, x_dev_ptr, in_features, x_dtype) == 0)

    def run_topk(self, x_dev_ptr: int, in_features: int, k: int, x_dtype: int = 0, weight: "Weight | None" = None) -> None:
        """Enqueues one forward of the candidate form: k (value, row) pairs per rank cross the links."""
        _check(lib().b200h_head_run_topk(self.h, weight.h if weight is not None else None, x_dev_ptr, in_features, x_dtype, k) == 0)

    def top(self, k: int):
        """Synchronises the device and returns (values, rows) of the latest run_topk, best first."""
        v, r = np.empty(k, np.float32), np.empty(k, np.int32)
        _check(lib().b200h_head_top_to_host(self.h, v.ctypes.data, r.ctypes.data, k) == 0)
        return v, r

    def top_rows_ptr(self) -> int:
        return int(lib().b200h_head_top_rows(self.h))

    def logits_ptr(self) -> int:
        return int(lib().b200h_head_logits(self.h))

    def calls(self) -> int:
        return int(lib().b200h_head_calls(self.h))

    def logits(self) -> np.ndarray:
        """Synchronises the device and returns the latest full result vector."""
        out = np.empty(self.total_rows, np.float32)
        _check(lib().b200h_head_logits_to_host(self.h, out.ctypes.data) == 0)
        return out

    def close(self):
        if self.h:
            lib().b200h_head_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass

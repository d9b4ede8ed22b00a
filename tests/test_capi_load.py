"""The C-ABI library loads on a machine without a GPU and exports every symbol
that include/b200q.h declares; device-free entry points answer correctly and
compute entry points fail with a CUDA error instead of falling back."""
import ctypes
import os
import re

import pytest

from brotensor_b200 import _capi as capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    if not os.path.exists(capi.LIB_PATH):
        from brotensor_b200 import build
        build.build_kernels()
    return capi.lib()


def test_every_declared_symbol_is_exported_and_bound(L):
    hdr = open(os.path.join(ROOT, "include", "b200q.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    declared = set(re.findall(r"\b((?:b200q|brotensor)_\w+)\s*\(", hdr))
    assert declared, "no declarations parsed"
    bound = {name for name, _, _ in capi.SYMBOLS}
    assert declared == bound
    for name in declared:
        assert getattr(L, name) is not None


def test_device_free_entry_points(L):
    assert L.b200q_abi_version() == 1
    assert (L.b200q_block_elems(capi.Q4_K), L.b200q_block_bytes(capi.Q4_K)) == (256, 144)
    assert (L.b200q_block_elems(capi.Q6_K), L.b200q_block_bytes(capi.Q6_K)) == (256, 210)
    assert (L.b200q_block_elems(capi.Q8_0), L.b200q_block_bytes(capi.Q8_0)) == (32, 34)
    assert L.b200q_block_elems(7) == 0
    assert L.b200q_packed_bytes(capi.Q4_K, 4096, 4096) == 9437184
    assert L.b200q_packed_bytes(capi.Q6_K, 128256, 4096) == 430940160
    assert L.b200q_packed_bytes(capi.Q8_0, 14336, 4096) == 62390272
    assert L.b200q_packed_bytes(capi.Q4_K, 4, 100) == 0
    assert L.b200q_status_str(capi.ERR_TIMEOUT) == b"device-side wait timed out"


def test_argument_validation_needs_no_device(L):
    buf = (ctypes.c_char * 4096)()
    p = ctypes.addressof(buf)
    p16 = (p + 15) & ~15
    assert L.b200q_gemv(99, p16, p16, capi.F32, None, p16, capi.F32, 1, 4, 256, None) == capi.ERR_BAD_ARG
    assert b"unknown block format" in L.b200q_last_error()
    assert L.b200q_gemv(capi.Q4_K, p16, p16, capi.F32, None, p16, capi.F32, 1, 4, 100, None) == capi.ERR_BAD_ARG
    assert L.b200q_gemv(capi.Q4_K, p16, p16, 3, None, p16, capi.F32, 1, 4, 256, None) == capi.ERR_BAD_ARG
    assert L.b200q_gemv(capi.Q4_K, p16, p16, capi.F32, None, p16, capi.F32, 9, 4, 256, None) == capi.ERR_UNSUPPORTED
    assert L.b200q_gemv(capi.Q4_K, None, p16, capi.F32, None, p16, capi.F32, 1, 4, 256, None) == capi.ERR_BAD_ARG
    assert L.b200q_gemv(capi.Q4_K, p16, p16 + 4, capi.F32, None, p16, capi.F32, 1, 4, 256, None) == capi.ERR_BAD_ARG
    # the sharded form checks its rank / row arguments before it touches the device
    tab = (ctypes.c_void_p * 8)(*([p16] * 8))
    sh = lambda rows, off, total, rank, world: L.b200q_gemv_shard(capi.Q4_K, p16, p16, capi.F32, None, rows, 256, off,
                                                                  total, rank, world, tab, p16, None)
    assert sh(4, 0, 4, 2, 2) == capi.ERR_BAD_ARG and b"rank 2 of 2" in L.b200q_last_error()
    assert sh(4, 0, 4, 0, 9) == capi.ERR_BAD_ARG
    assert sh(4, 2, 4, 0, 1) == capi.ERR_BAD_ARG and b"do not lie in" in L.b200q_last_error()
    assert sh(0, 0, 4, 0, 1) == capi.ERR_UNSUPPORTED
    # empty problems are legal and touch nothing
    assert L.b200q_gemv(capi.Q4_K, None, None, capi.F32, None, None, capi.F32, 0, 4, 256, None) == capi.OK
    assert L.b200q_dequant(capi.Q8_0, None, None, capi.F16, 0, 32, None) == capi.OK
    assert L.b200q_set_option(b"no_such_key", 1) == capi.ERR_BAD_ARG


def test_compute_fails_loudly_without_a_gpu(L):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    buf = (ctypes.c_char * 4096)()
    p16 = (ctypes.addressof(buf) + 15) & ~15
    rc = L.b200q_gemv(capi.Q4_K, p16, p16, capi.F32, None, p16, capi.F32, 1, 4, 256, None)
    assert rc == capi.ERR_CUDA
    assert b"CUDA error" in L.b200q_last_error()

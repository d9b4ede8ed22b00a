"""The C++ host layer (Tensor / dispatch / nine ops / GGUF reader): its own C++ test
executable, plus a cross-check of the GGUF reader against the reference's reader
(oracle/_ref, when built) on files written here."""
import ctypes as C
import os
import struct
import subprocess

import numpy as np
import pytest

import oracle
from brotensor_b200 import synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "brotensor_b200", "lib")


@pytest.fixture(scope="module")
def built():
    import importlib.util
    spec = importlib.util.spec_from_file_location("build_host_tests", os.path.join(ROOT, "tests", "cpp", "build_host_tests.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build()


def run_host_tests(exe, mode):
    r = subprocess.run([exe, mode], capture_output=True, text=True, timeout=600)
    print(r.stdout[-3000:], r.stderr[-2000:])
    assert r.returncode == 0, r.stdout[-2000:]
    return r.stdout


def test_host_layer_cpu_cases(built):
    out = run_host_tests(built, "cpu")
    assert "OK (0 failures)" in out


@pytest.mark.gpu
def test_host_layer_gpu_cases(built):
    out = run_host_tests(built, "gpu")
    assert "OK (0 failures)" in out and "skipping" not in out


def _gguf_bytes(tensors, align=32, version=3, meta=()):
    """tensors: list of (name, dims innermost-first, ggml_type, payload bytes)."""
    b = bytearray()
    b += struct.pack("<IIQQ", 0x46554747, version, len(tensors), len(meta) + 1)
    key = b"general.alignment"
    b += struct.pack("<Q", len(key)) + key + struct.pack("<II", 4, align)
    for k, v in meta:
        kb, vb = k.encode(), v.encode()
        b += struct.pack("<Q", len(kb)) + kb + struct.pack("<IQ", 8, len(vb)) + vb
    off = 0
    offs = []
    for name, dims, typ, payload in tensors:
        nb = name.encode()
        b += struct.pack("<Q", len(nb)) + nb + struct.pack("<I", len(dims))
        for d in dims:
            b += struct.pack("<Q", d)
        b += struct.pack("<IQ", typ, off)
        offs.append(off)
        off += (len(payload) + align - 1) // align * align
    while len(b) % align:
        b += b"\0"
    for (name, dims, typ, payload), o in zip(tensors, offs):
        b += payload + b"\0" * ((align - len(payload) % align) % align)
    return bytes(b)


@pytest.fixture(scope="module")
def hostlib(built):
    L = C.CDLL(os.path.join(LIB, "libbrotensor_b200.so"))
    L.b200h_last_error.restype = C.c_char_p
    L.b200h_gguf_open.restype = C.c_void_p
    L.b200h_gguf_open.argtypes = [C.c_char_p]
    for f in ("b200h_gguf_close", "b200h_gguf_tensor_count", "b200h_gguf_alignment", "b200h_gguf_version"):
        getattr(L, f).argtypes = [C.c_void_p]
    L.b200h_gguf_tensor.argtypes = [C.c_void_p, C.c_int, C.c_char_p, C.c_int, C.POINTER(C.c_longlong), C.POINTER(C.c_int),
                                    C.POINTER(C.c_uint), C.POINTER(C.c_int), C.POINTER(C.c_int),
                                    C.POINTER(C.c_ulonglong), C.POINTER(C.c_longlong), C.POINTER(C.c_ulonglong)]
    L.b200h_gguf_upload_rows.restype = C.c_void_p
    L.b200h_gguf_upload_rows.argtypes = [C.c_void_p] + [C.c_int] * 6
    L.b200h_tensor_to_host.argtypes = [C.c_void_p, C.c_void_p]
    L.b200h_tensor_free.argtypes = [C.c_void_p]
    L.b200h_shape_to_2d.argtypes = [C.POINTER(C.c_longlong), C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]
    assert L.b200h_init() >= 0
    return L


def _ours(L, path):
    h = L.b200h_gguf_open(path.encode())
    assert h, L.b200h_last_error()
    rows = []
    for i in range(L.b200h_gguf_tensor_count(h)):
        name = C.create_string_buffer(256)
        shape = (C.c_longlong * 8)()
        nd, typ, dt, sup = C.c_int(), C.c_uint(), C.c_int(), C.c_int()
        nb, ne, off = C.c_ulonglong(), C.c_longlong(), C.c_ulonglong()
        assert L.b200h_gguf_tensor(h, i, name, 256, shape, C.byref(nd), C.byref(typ), C.byref(dt), C.byref(sup),
                                   C.byref(nb), C.byref(ne), C.byref(off)) == 0
        rows.append((name.value.decode(), tuple(shape[:nd.value]), typ.value, dt.value, sup.value, nb.value, ne.value, off.value))
    meta = (L.b200h_gguf_alignment(h), L.b200h_gguf_version(h))
    return h, rows, meta


def test_gguf_reader_agrees_with_reference_reader(hostlib, tmp_path):
    r = oracle.ref()
    if r is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    q4 = synth.make_blocks(synth.Q4_K, 8, 512, seed=1).tobytes()
    q6 = synth.make_blocks(synth.Q6_K, 6, 256, seed=2).tobytes()
    q8 = synth.make_blocks(synth.Q8_0, 3, 64, seed=3).tobytes()
    f32 = np.arange(24, dtype=np.float32).tobytes()
    for align, version in ((32, 3), (64, 2), (256, 3)):
        data = _gguf_bytes([("blk.0.q", [512, 8], 12, q4), ("blk.0.down", [256, 2, 3], 14, q6),
                            ("emb", [64, 3], 8, q8), ("norm", [24], 0, f32), ("odd", [4], 77, b"")],
                           align=align, version=version, meta=[("general.name", "synthetic")])
        p = str(tmp_path / f"a{align}.gguf")
        open(p, "wb").write(data)
        h, ours, meta = _ours(hostlib, p)
        err = C.create_string_buffer(256)
        n = r.lib.ref_gguf_open(p.encode(), err, 256)
        assert n == len(ours), err.value
        assert meta == (r.lib.ref_gguf_alignment(), r.lib.ref_gguf_version())
        for i, row in enumerate(ours):
            name = C.create_string_buffer(256)
            shape = (C.c_int64 * 8)()
            nd, typ, dt, sup = C.c_int(), C.c_uint32(), C.c_int(), C.c_int()
            nb, ne, off = C.c_uint64(), C.c_int64(), C.c_uint64()
            r.lib.ref_gguf_tensor(i, name, 256, shape, C.byref(nd), C.byref(typ), C.byref(dt), C.byref(sup),
                                  C.byref(nb), C.byref(ne), C.byref(off))
            assert row == (name.value.decode(), tuple(shape[:nd.value]), typ.value, dt.value, sup.value, nb.value,
                           ne.value, off.value)
        r.lib.ref_gguf_close()
        # a row shard of the Q4_K tensor is a contiguous byte range, content unchanged
        t = hostlib.b200h_gguf_upload_rows(h, 0, 8, 512, 2, 6, -1)
        assert t, hostlib.b200h_last_error()
        buf = np.empty(4 * 2 * 144, np.uint8)
        assert hostlib.b200h_tensor_to_host(t, buf.ctypes.data) == 0
        assert buf.tobytes() == q4[2 * 288:6 * 288]
        hostlib.b200h_tensor_free(t)
        hostlib.b200h_gguf_close(h)


def test_shape_to_2d_agrees_with_reference(hostlib):
    r = oracle.ref()
    if r is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    for shape in ([7], [256, 4], [256, 2, 3], [32, 1, 1, 5], [0, 3], [1 << 40, 2], [2, 70000, 70000], []):
        a = (C.c_longlong * max(1, len(shape)))(*shape)
        b = (C.c_int64 * max(1, len(shape)))(*shape)
        r1, c1, r2, c2 = C.c_int(), C.c_int(), C.c_int(), C.c_int()
        err = C.create_string_buffer(256)
        ok_ours = hostlib.b200h_shape_to_2d(a, len(shape), C.byref(r1), C.byref(c1)) == 0
        ok_ref = r.lib.ref_shape_to_2d(b, len(shape), C.byref(r2), C.byref(c2), err, 256) == 0
        assert ok_ours == ok_ref
        if ok_ours:
            assert (r1.value, c1.value) == (r2.value, c2.value)
        else:
            assert err.value.decode() == hostlib.b200h_last_error().decode()


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,N,K", [(synth.Q4_K, 1024, 512), (synth.Q6_K, 256, 2048), (synth.Q8_0, 384, 256)])
def test_session_enqueue_with_pinned_buffers_equals_blocking_run(built, fmt, N, K):
    """The non-blocking round trip (page-locked host buffers, one sync) gives the blocking one's bytes."""
    import torch
    from brotensor_b200 import hostapi
    hostapi.init()
    w = hostapi.Weight(fmt, synth.make_blocks(fmt, N, K, seed=11), N, K, 0)
    sess = hostapi.Session(w, 1, 0, 0)
    outs = []
    for i in range(3):
        xh = synth.make_activations(1, K, seed=30 + i)
        ref = sess.run(xh).copy().reshape(-1)
        xp = torch.from_numpy(xh.reshape(-1)).pin_memory()
        yp = torch.zeros(N, dtype=torch.float32).pin_memory()
        sess.enqueue(xp.data_ptr(), yp.data_ptr())
        hostapi.sync(0)
        assert np.array_equal(yp.numpy(), ref)
        outs.append(ref)
    assert not np.array_equal(outs[0], outs[1])
    sess.close()


@pytest.mark.gpu
def test_captured_step_replays_with_new_inputs(built):
    """CudaGraphCapture around two ops with their host round trips; the replay sees what is in
    the pinned input buffers at launch time."""
    import torch
    from brotensor_b200 import hostapi
    hostapi.init()
    specs = [(synth.Q4_K, 512, 512), (synth.Q6_K, 256, 2048)]
    ws = [hostapi.Weight(f, synth.make_blocks(f, N, K, seed=5 + i), N, K, 0) for i, (f, N, K) in enumerate(specs)]
    ss = [hostapi.Session(w, 1, 0, 0) for w in ws]
    xp = [torch.zeros(K, dtype=torch.float32).pin_memory() for _, _, K in specs]
    yp = [torch.zeros(N, dtype=torch.float32).pin_memory() for _, N, _ in specs]

    def enqueue():
        for s, x, y in zip(ss, xp, yp):
            s.enqueue(x.data_ptr(), y.data_ptr())

    enqueue()                     # warm-up: outputs allocated, kernels configured
    hostapi.sync(0)
    with hostapi.Graph.capture() as g:
        enqueue()
    for rep in range(3):
        xs = [synth.make_activations(1, K, seed=70 + rep + i).reshape(-1) for i, (_, _, K) in enumerate(specs)]
        for x, v in zip(xp, xs):
            x.copy_(torch.from_numpy(v))
        g.launch()
        hostapi.sync(0)
        for s, v, y in zip(ss, xs, yp):
            assert np.array_equal(y.numpy(), s.run(v.reshape(1, -1)).reshape(-1)), f"replay {rep}"
    g.close()


@pytest.mark.gpu
def test_layer_set_one_copy_in_one_copy_out(built):
    """LayerSet: activations and results of several GEMVs in one arena each; a captured step with
    one copy in and one copy out gives every op's blocking result."""
    import torch
    from brotensor_b200 import hostapi
    hostapi.init()
    specs = [(synth.Q4_K, 512, 512), (synth.Q4_K, 100, 256), (synth.Q6_K, 256, 2048), (synth.Q8_0, 96, 128)]
    ws = [hostapi.Weight(f, synth.make_blocks(f, N, K, seed=9 + i), N, K, 0) for i, (f, N, K) in enumerate(specs)]
    L = hostapi.LayerSet(ws)
    assert all(o % 256 == 0 for o in L.x_off + L.y_off)
    xa = torch.zeros(L.x_bytes, dtype=torch.uint8).pin_memory()
    ya = torch.zeros(L.y_bytes, dtype=torch.uint8).pin_memory()
    L.enqueue(xa.data_ptr(), ya.data_ptr())
    hostapi.sync(0)
    with hostapi.Graph.capture() as g:
        L.enqueue(xa.data_ptr(), ya.data_ptr())
    ss = [hostapi.Session(w, 1, 0, 0) for w in ws]
    for rep in range(2):
        xs = [synth.make_activations(1, K, seed=90 + rep + i) for i, (_, _, K) in enumerate(specs)]
        for off, v in zip(L.x_off, xs):
            xa[off:off + v.nbytes] = torch.from_numpy(v.reshape(-1).view(np.uint8))
        g.launch()
        hostapi.sync(0)
        for s, v, off, (_, N, _) in zip(ss, xs, L.y_off, specs):
            got = ya[off:off + 4 * N].numpy().view(np.float32)
            assert np.array_equal(got, s.run(v).reshape(-1)), f"replay {rep}"
    g.close()
    L.close()


@pytest.mark.gpu
def test_repack_weights_keeps_every_op_bit_identical(built):
    """brotensor_b200::repack_weights regroups a Q6_K weight on the device in place: the ops
    find the layout through the storage record and return the raw layout's bits; unpack_weights
    restores the GGUF bytes; formats without a regrouped form are left alone."""
    from brotensor_b200 import hostapi
    hostapi.init()
    N, K = 320, 4096
    blocks = synth.make_blocks(synth.Q6_K, N, K, seed=5)
    w = hostapi.Weight(synth.Q6_K, blocks, N, K, 0)
    assert not w.repacked
    x1 = synth.make_activations(1, K, seed=1)
    x4 = synth.make_activations(4, K, seed=2)
    x40 = synth.make_activations(40, K, seed=3)
    s1, s40 = hostapi.Session(w, 1, 0, 0), hostapi.Session(w, 40, 0, 0)
    raw = dict(deq=w.dequant(1).copy(), y1=s1.run(x1).copy(), y40=s40.run(x40).copy())
    assert w.repack() is True and w.repacked
    with pytest.raises(RuntimeError, match="regrouped device layout"):
        w.raw_bytes()                                         # regrouped bytes never reach host code by accident
    assert np.array_equal(w.dequant(1), raw["deq"])
    assert np.array_equal(s1.run(x1), raw["y1"])
    assert np.array_equal(s40.run(x40), raw["y40"])
    s4 = hostapi.Session(w, 4, 0, 0)
    y4 = s4.run(x4).copy()
    assert w.repack() is True                                  # a second call changes nothing
    assert np.array_equal(s1.run(x1), raw["y1"])
    w.unpack()
    assert not w.repacked and np.array_equal(w.raw_bytes(), blocks)
    assert np.array_equal(s1.run(x1), raw["y1"])
    ref4 = s4.run(x4)
    assert np.abs(ref4 - y4).max() <= 2e-3 * np.abs(ref4).max()  # four rows: different kernels per layout
    for s in (s1, s4, s40):
        s.close()
    w.close()
    # a weight that reuses the freed storage starts in the GGUF layout; Q4_K has no regrouped form
    w2 = hostapi.Weight(synth.Q6_K, blocks, N, K, 0)
    assert not w2.repacked
    w2.close()
    w3 = hostapi.Weight(synth.Q4_K, synth.make_blocks(synth.Q4_K, 64, 512, seed=1), 64, 512, 0)
    assert w3.repack() is False and not w3.repacked
    w3.close()

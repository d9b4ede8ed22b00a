"""Generates the golden fixtures in this folder from brotensor's own host
reference (oracle/_ref/libref.so, compiled from the reference tree by
oracle/Makefile). Run it where the reference tree is present:

    python tests/golden/make_golden.py

Each ``<fmt>_parity.npz`` replays the seeded inputs of the reference's parity
test for that format (tests/test_q4k_parity.cpp, test_q6k_parity.cpp,
test_q8_0_parity.cpp): weights U(-0.5,0.5) quantized by the reference quantizer,
decoded by the reference block decoder, activations U(-0.3,0.3), bias
U(-0.1,0.1), all drawn in the tests' order from std::mt19937 with the tests'
seeds, and the expected outputs from the reference's decode + sequential FP32
dot. ``prefill_lcg.npz`` replays tests/test_quant_prefill_parity.cpp's LCG byte
blocks. ``kat.npz`` holds known answers for the 6-bit scale packing and the
fp16/bf16 conversions.
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import oracle  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
SEEDS = {oracle.Q4_K: 0xC0FFEE, oracle.Q6_K: 0xBADBEEF, oracle.Q8_0: 0xCAFEBABE}
NAMES = {oracle.Q4_K: "q4k", oracle.Q6_K: "q6k", oracle.Q8_0: "q8_0"}


def parity_case(r, fmt):
    OUT, IN, B = 64, 256, 4
    r.seed(SEEDS[fmt])
    out = {}
    Wf = r.uniform(-0.5, 0.5, OUT * IN).reshape(OUT, IN)
    Wq = r.quantize(fmt, Wf)
    Wd = r.dequant_f32(fmt, Wq, OUT, IN)
    x = r.uniform(-0.3, 0.3, IN)
    bias = r.uniform(-0.1, 0.1, OUT)
    X = r.uniform(-0.3, 0.3, B * IN).reshape(B, IN)
    out.update(A_W=Wq, A_Wdeq=Wd, A_Wdeq_fp16=r.fp32_to_fp16(Wd).reshape(OUT, IN),
               B_x=x, B_y=r.matmul(fmt, Wq, x[None, :])[0], C_bias=bias,
               C_y=r.matmul(fmt, Wq, x[None, :])[0] + bias,  # the test adds bias to y_ref (:308)
               D_X=X, D_Y=r.matmul(fmt, Wq, X))
    # E/F/G continue on the same generator, weights first then activations.
    for label, (o2, i2, b2) in {"E": (64, 512, 16), "F": (64, 512, 2), "G": (128, 1024, 32)}.items():
        Wf2 = r.uniform(-0.5, 0.5, o2 * i2).reshape(o2, i2)
        Wq2 = r.quantize(fmt, Wf2)
        X2 = r.uniform(-0.3, 0.3, b2 * i2).reshape(b2, i2)
        out[f"{label}_W"] = Wq2
        out[f"{label}_X"] = X2
        out[f"{label}_Y"] = r.matmul(fmt, Wq2, X2)
    return out


def prefill_lcg_case(r, fmt):
    """96 x (3 blocks) weights from the test's byte LCG with pinned fp16 scales, B=16."""
    be, bb = oracle.BLOCK_ELEMS[fmt], oracle.BLOCK_BYTES[fmt]
    OUT, IN, B = 96, be * 3, 16
    nb = OUT * 3
    n = nb * bb
    lcg = 0x1234567
    raw = np.empty(n, np.uint8)
    for i in range(n):
        lcg = (lcg * 1664525 + 1013904223) & 0xFFFFFFFF
        raw[i] = lcg >> 24
    blk = raw.reshape(nb, bb)

    def put(off, v):
        h = int(r.fp32_to_fp16(np.float32(v))[0])
        blk[:, off] = h & 0xFF
        blk[:, off + 1] = h >> 8

    if fmt == oracle.Q4_K:
        put(0, 0.02)
        put(2, 0.008)
    elif fmt == oracle.Q8_0:
        put(0, 0.01)
    else:
        put(bb - 2, 0.01)
    lcg = 0xABCD
    vals = np.empty(B * IN + OUT, np.float32)
    for i in range(vals.size):
        lcg = (lcg * 1664525 + 1013904223) & 0xFFFFFFFF
        vals[i] = np.float32(np.float32(lcg >> 8) / np.float32(1 << 24)) * np.float32(0.6) - np.float32(0.3)
    Xh = r.fp32_to_fp16(vals[: B * IN]).reshape(B, IN)
    bh = r.fp32_to_fp16(vals[B * IN:])
    Xf = r.fp16_to_fp32(Xh).reshape(B, IN)
    bf = r.fp16_to_fp32(bh)
    W = blk.reshape(-1)
    return {"W": W, "X_fp16": Xh, "bias_fp16": bh, "Y": r.matmul(fmt, W, Xf), "Y_bias": r.matmul(fmt, W, Xf, bf)}


def main():
    r = oracle.ref()
    assert r is not None, "oracle/_ref/libref.so missing: run `make -C oracle` where the reference tree exists"
    for fmt, name in NAMES.items():
        np.savez_compressed(os.path.join(HERE, f"{name}_parity.npz"), **parity_case(r, fmt))
    pre = {}
    for fmt, name in NAMES.items():
        for k, v in prefill_lcg_case(r, fmt).items():
            pre[f"{name}_{k}"] = v
    np.savez_compressed(os.path.join(HERE, "prefill_lcg.npz"), **pre)

    rng = np.random.default_rng(7)
    sc = rng.integers(0, 64, size=(256, 8), dtype=np.uint8)
    m = rng.integers(0, 64, size=(256, 8), dtype=np.uint8)
    packed = np.zeros((256, 12), np.uint8)
    import ctypes as C
    u8p = C.POINTER(C.c_uint8)
    for i in range(256):
        r.lib.ref_q4k_pack_sc_m(packed[i].ctypes.data_as(u8p), sc[i].ctypes.data_as(u8p), m[i].ctypes.data_as(u8p))
    # unpack of arbitrary bytes (all 96 bits random) through the reference unpacker
    rnd12 = rng.integers(0, 256, size=(256, 12), dtype=np.uint8)
    usc = np.zeros((256, 8), np.uint8)
    um = np.zeros((256, 8), np.uint8)
    for i in range(256):
        r.lib.ref_q4k_unpack_sc_m(rnd12[i].ctypes.data_as(u8p), usc[i].ctypes.data_as(u8p), um[i].ctypes.data_as(u8p))
    f = np.concatenate([
        rng.standard_normal(2000).astype(np.float32) * np.float32(3.0),
        (rng.standard_normal(500) * 1e-6).astype(np.float32),  # fp16 subnormal range
        np.array([0.0, -0.0, 1.0, -1.0, 65504.0, 65519.9, 65520.0, 1e-8, 5.9604645e-8, 2.9802322e-8,
                  6.1035156e-5, 6.0975552e-5, 1.0009766, 1.00048828125, 1.0014648, np.inf, -np.inf], np.float32),
    ])
    all16 = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    np.savez_compressed(os.path.join(HERE, "kat.npz"), sc=sc, m=m, packed=packed, rnd12=rnd12, usc=usc, um=um,
                        f32=f, f32_as_fp16=r.fp32_to_fp16(f), f32_as_bf16=r.fp32_to_bf16(f),
                        fp16_all_as_f32=r.fp16_to_fp32(all16))
    for fn in sorted(os.listdir(HERE)):
        if fn.endswith(".npz"):
            print(fn, os.path.getsize(os.path.join(HERE, fn)))


if __name__ == "__main__":
    main()

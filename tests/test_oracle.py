"""Pins the CPU oracle (oracle/b200q_oracle.c) to brotensor's own host reference:
against the committed golden vectors always, and against the reference functions
themselves (oracle/_ref) on fresh random blocks wherever that library exists."""
import numpy as np
import pytest

import oracle
from brotensor_b200 import synth

FMTS = [(oracle.Q4_K, "q4k"), (oracle.Q6_K, "q6k"), (oracle.Q8_0, "q8_0")]


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


@pytest.mark.parametrize("fmt,name", FMTS)
def test_decode_matches_golden_bitwise(fmt, name, golden, cpu_oracle):
    g = golden(name + "_parity")
    got = cpu_oracle.dequant_f32(fmt, g["A_W"], 64, 256)
    assert np.array_equal(bits(got), bits(g["A_Wdeq"]))
    got16 = cpu_oracle.dequant_16(fmt, g["A_W"], 64, 256, 1)
    assert np.array_equal(got16, g["A_Wdeq_fp16"])


@pytest.mark.parametrize("fmt,name", FMTS)
def test_matmul_matches_golden(fmt, name, golden, cpu_oracle):
    g = golden(name + "_parity")
    y = cpu_oracle.matmul(fmt, g["A_W"], g["B_x"][None, :])[0]
    # Same decode, same sequential order; only FMA contraction in the reference
    # build can differ, a few ulp of a K=256 dot product.
    assert np.abs(y - g["B_y"]).max() < 1e-5
    yb = cpu_oracle.matmul(fmt, g["A_W"], g["B_x"][None, :], bias=g["C_bias"])[0]
    assert np.abs(yb - g["C_y"]).max() < 1e-5
    Y = cpu_oracle.matmul(fmt, g["A_W"], g["D_X"], threads=3)
    assert np.abs(Y - g["D_Y"]).max() < 1e-5
    for label in "EFG":
        Y = cpu_oracle.matmul(fmt, g[label + "_W"], g[label + "_X"], threads=4)
        assert oracle.rel_l2(Y, g[label + "_Y"]) < 1e-6


@pytest.mark.parametrize("fmt,name", FMTS)
def test_prefill_lcg_blocks(fmt, name, golden, cpu_oracle):
    """Arbitrary block bytes (every bit pattern of scales and quants) with pinned fp16 scales."""
    g = golden("prefill_lcg")
    X = g[name + "_X_fp16"].view(np.float16).astype(np.float32)
    b = g[name + "_bias_fp16"].view(np.float16).astype(np.float32)
    assert oracle.rel_l2(cpu_oracle.matmul(fmt, g[name + "_W"], X), g[name + "_Y"]) < 1e-6
    assert oracle.rel_l2(cpu_oracle.matmul(fmt, g[name + "_W"], X, bias=b), g[name + "_Y_bias"]) < 1e-6


def test_scale_pack_unpack_kat(golden, cpu_oracle):
    k = golden("kat")
    for i in range(256):
        assert np.array_equal(cpu_oracle.q4k_pack_sc_m(k["sc"][i], k["m"][i]), k["packed"][i])
        sc, m = cpu_oracle.q4k_unpack_sc_m(k["packed"][i])
        assert np.array_equal(sc, k["sc"][i]) and np.array_equal(m, k["m"][i])
        sc, m = cpu_oracle.q4k_unpack_sc_m(k["rnd12"][i])
        assert np.array_equal(sc, k["usc"][i]) and np.array_equal(m, k["um"][i])


def test_float_conversions_kat(golden, cpu_oracle):
    k = golden("kat")
    # The reference's host converter (src/tensor.cpp:184-190) rounds ties in the fp16
    # subnormal range upward; the oracle rounds them to even like the reference's
    # device kernels (__float2half_rn, src/cuda/q4k.cu:95). Decoded weights in that
    # range are multiples of 2^-24, so no tie can occur on this path; the one tie in
    # the vector (2^-25) is checked separately.
    tie = k["f32"] == np.float32(2.0 ** -25)
    assert tie.sum() == 1 and k["f32_as_fp16"][tie][0] == 1 and cpu_oracle.fp32_to_fp16(k["f32"][tie])[0] == 0
    assert np.array_equal(cpu_oracle.fp32_to_fp16(k["f32"])[~tie], k["f32_as_fp16"][~tie])
    assert np.array_equal(cpu_oracle.fp32_to_bf16(k["f32"]), k["f32_as_bf16"])
    all16 = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    got = cpu_oracle.fp16_to_fp32(all16)
    want = k["fp16_all_as_f32"]
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(bits(got)[~nan], bits(want)[~nan])
    # numpy's own converters agree too (used by the generators)
    assert np.array_equal(k["f32"].astype(np.float16).view(np.uint16)[~tie], k["f32_as_fp16"][~tie])
    finite = np.isfinite(k["f32"])
    assert np.array_equal(synth.to_bf16_bits(k["f32"][finite]), k["f32_as_bf16"][finite])


@pytest.mark.parametrize("fmt,name", FMTS)
def test_against_reference_library_on_synthetic_blocks(fmt, name, cpu_oracle):
    r = oracle.ref()
    if r is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    rows, K = 48, 1024
    W = synth.make_blocks(fmt, rows, K, seed=11)
    assert np.array_equal(bits(cpu_oracle.dequant_f32(fmt, W, rows, K)), bits(r.dequant_f32(fmt, W, rows, K)))
    X = synth.make_activations(3, K, seed=11)
    assert oracle.rel_l2(cpu_oracle.matmul(fmt, W, X, threads=2), r.matmul(fmt, W, X)) < 1e-6


@pytest.mark.parametrize("fmt,name", FMTS)
def test_oracle_edge_cases(fmt, name, cpu_oracle):
    be = oracle.BLOCK_ELEMS[fmt]
    # zero rows and zero activation rows are legal and produce empty outputs
    W = synth.make_blocks(fmt, 0, be, seed=1)
    assert cpu_oracle.dequant_f32(fmt, W, 0, be).shape == (0, be)
    W = synth.make_blocks(fmt, 5, be, seed=1)
    assert cpu_oracle.matmul(fmt, W, np.zeros((0, be), np.float32)).shape == (0, 5)
    # all-zero blocks decode to zero; extreme scale fields stay finite
    Z = np.zeros(oracle.BLOCK_BYTES[fmt] * 2, np.uint8)
    assert not cpu_oracle.dequant_f32(fmt, Z, 2, be).any()
    # thread count never changes results
    W = synth.make_blocks(fmt, 37, be * 2, seed=3)
    X = synth.make_activations(2, be * 2, seed=3)
    assert np.array_equal(cpu_oracle.matmul(fmt, W, X, threads=1), cpu_oracle.matmul(fmt, W, X, threads=8))


def test_decode_is_exact_in_fp32():
    """Both products are exact in fp32 and the one subtraction is correctly rounded,
    so evaluation order and FMA contraction cannot change the decoded weight:
    compare against float64 arithmetic (exact here) rounded once to fp32."""
    o = oracle.cpu()
    W = synth.make_blocks(oracle.Q4_K, 64, 1024, seed=5)
    got = o.dequant_f32(oracle.Q4_K, W, 64, 1024)
    blk = W.reshape(-1, 144)
    d = blk[:, 0:2].copy().view(np.float16).astype(np.float64)[:, 0]
    dm = blk[:, 2:4].copy().view(np.float16).astype(np.float64)[:, 0]
    want = np.empty((blk.shape[0], 256))
    for i in range(blk.shape[0]):
        sc, m = o.q4k_unpack_sc_m(blk[i, 4:16])
        qs = blk[i, 16:]
        for s in range(8):
            q = qs[(s >> 1) * 32:(s >> 1) * 32 + 32]
            nib = (q >> 4) if (s & 1) else (q & 15)
            want[i, s * 32:(s + 1) * 32] = d[i] * float(sc[s]) * nib - dm[i] * float(m[s])
    assert np.array_equal(bits(got.reshape(-1, 256)), bits(want.astype(np.float32)))

"""GPU parity tests: every result of the CUDA library (through the C-ABI) against
the CPU oracle on the same seeded inputs and against the committed golden vectors.

Tolerances. Block decode: bit-exact (FP32, and FP16/BF16 = round-to-nearest-even
of it). Matmul: relative L2 error <= 2e-3 against the FP32 host reference — the
bound the benchmark specification states — plus the reference tests' own absolute
bounds (5e-2 / 1e-1) on their own cases.
"""
import numpy as np
import pytest
import torch

import oracle
from brotensor_b200 import ops, synth

pytestmark = pytest.mark.gpu

REL_L2 = 2e-3
FMTS = [(oracle.Q4_K, "q4k"), (oracle.Q6_K, "q6k"), (oracle.Q8_0, "q8_0")]
TORCH_DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host_f32(t):
    return t.float().cpu().numpy()


def as_dtype_np(x, name):
    """fp32 array rounded to the activation dtype and back (what the kernel sees)."""
    t = torch.from_numpy(np.ascontiguousarray(x)).to(TORCH_DT[name])
    return t, t.float().numpy()


# (gemv_path, pipelines): plain-load kernel; automatic routing with one / two
# producer-consumer pipelines per CTA in the integer-dot kernel
PATHS = [(1, 2), (0, 1), (0, 2)]


def set_path(path):
    ops.set_option("gemv_path", path[0])
    ops.set_option("gemv_groups", path[1])


@pytest.fixture(autouse=True)
def _clean_state():
    set_path((0, 2))
    yield
    set_path((0, 2))
    assert ops.device_status() == 0


# ---------------------------------------------------------------- block decode

@pytest.mark.parametrize("fmt,name", FMTS)
def test_dequant_bit_exact_golden(fmt, name, golden):
    g = golden(name + "_parity")
    W = dev(g["A_W"])
    f32 = ops.dequant(fmt, W, 64, 256, torch.float32).cpu().numpy()
    assert np.array_equal(f32.view(np.uint32), g["A_Wdeq"].view(np.uint32))
    f16 = ops.dequant(fmt, W, 64, 256, torch.float16).cpu().numpy()
    assert np.array_equal(f16.view(np.uint16), g["A_Wdeq_fp16"])


@pytest.mark.parametrize("fmt,name", FMTS)
@pytest.mark.parametrize("rows,K", [(1, 256), (3, 512), (257, 1024), (148 * 16 + 5, 2048)])
def test_dequant_bit_exact_synthetic(fmt, name, rows, K, cpu_oracle):
    Wh = synth.make_blocks(fmt, rows, K, seed=rows + K)
    W = dev(Wh)
    want32 = cpu_oracle.dequant_f32(fmt, Wh, rows, K)
    got32 = ops.dequant(fmt, W, rows, K, torch.float32).cpu().numpy()
    assert np.array_equal(got32.view(np.uint32), want32.view(np.uint32))
    got16 = ops.dequant(fmt, W, rows, K, torch.float16).cpu().numpy()
    assert np.array_equal(got16.view(np.uint16), cpu_oracle.dequant_16(fmt, Wh, rows, K, 1))
    gotbf = ops.dequant(fmt, W, rows, K, torch.bfloat16).view(torch.int16).cpu().numpy()
    assert np.array_equal(gotbf.view(np.uint16), cpu_oracle.dequant_16(fmt, Wh, rows, K, 4))


def test_dequant_rows_beyond_grid_y_limit(cpu_oracle):
    """70 000 one-block rows: the reference regression case for gridDim.y > 65535
    (tests/test_q8_0_parity.cpp:296-361): full decode == decode of the two halves."""
    rows, K = 70000, 32
    Wh = synth.make_blocks(oracle.Q8_0, rows, K, seed=9)
    full = ops.dequant(oracle.Q8_0, dev(Wh), rows, K).cpu().numpy()
    h0 = rows // 2
    a = ops.dequant(oracle.Q8_0, dev(Wh[: h0 * 34]), h0, K).cpu().numpy()
    b = ops.dequant(oracle.Q8_0, dev(Wh[h0 * 34:]), rows - h0, K).cpu().numpy()
    assert np.array_equal(full.view(np.uint16), np.concatenate([a, b]).view(np.uint16))
    assert np.array_equal(full.view(np.uint16), cpu_oracle.dequant_16(oracle.Q8_0, Wh, rows, K, 1))


# ---------------------------------------------------------------- reference test cases

@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("fmt,name", FMTS)
def test_reference_parity_cases(fmt, name, path, golden):
    """Cases B, C, D, E, F, G of the reference parity tests with FP16 activations
    and FP16 outputs (the reference contract) and the reference's absolute bounds."""
    set_path(path)
    g = golden(name + "_parity")
    W = dev(g["A_W"])
    x = dev(g["B_x"]).half()
    y = ops.gemv(fmt, W, x, 64)
    assert y.dtype == torch.float16 and tuple(y.shape) == (1, 64)
    assert np.abs(host_f32(y)[0] - g["B_y"]).max() < 5e-2
    yb = ops.gemv(fmt, W, x, 64, bias=dev(g["C_bias"]).half())
    assert np.abs(host_f32(yb)[0] - g["C_y"]).max() < 5e-2
    Y = ops.linear(fmt, W, dev(g["D_X"]).half(), 64)
    assert np.abs(host_f32(Y) - g["D_Y"]).max() < 5e-2
    for label, tol in (("E", 5e-2), ("F", 5e-2), ("G", 1e-1)):
        X = g[label + "_X"]
        n = g[label + "_Y"].shape[1]
        Y = ops.linear(fmt, dev(g[label + "_W"]), dev(X).half(), n)
        assert np.abs(host_f32(Y) - g[label + "_Y"]).max() < tol
        # and the tight bound with FP32 activations / outputs
        Y32 = ops.linear(fmt, dev(g[label + "_W"]), dev(X), n)
        assert oracle.rel_l2(host_f32(Y32), g[label + "_Y"]) < REL_L2


@pytest.mark.parametrize("fmt,name", FMTS)
def test_prefill_lcg_case(fmt, name, golden):
    """tests/test_quant_prefill_parity.cpp: arbitrary block bytes, B=16, with and without bias."""
    g = golden("prefill_lcg")
    W = dev(g[name + "_W"])
    X = torch.from_numpy(g[name + "_X_fp16"].view(np.float16)).cuda()
    b = torch.from_numpy(g[name + "_bias_fp16"].view(np.float16)).cuda()
    Y = ops.linear(fmt, W, X, 96)
    Yb = ops.linear(fmt, W, X, 96, bias=b)
    for got, want in ((Y, g[name + "_Y"]), (Yb, g[name + "_Y_bias"])):
        err = np.abs(host_f32(got) - want)
        assert np.all(err <= 3e-2 + 5e-2 * np.abs(want))  # the reference test's bound (:133-145)
    Y32 = ops.linear(fmt, W, X, 96, out_dtype=torch.float32)
    assert oracle.rel_l2(host_f32(Y32), g[name + "_Y"]) < REL_L2


# ---------------------------------------------------------------- decode GEMV vs oracle

SHAPES = {
    oracle.Q4_K: [(1, 256), (7, 512), (17, 1024), (100, 4096), (1000, 2048), (148 * 16 + 3, 512)],
    oracle.Q6_K: [(1, 256), (7, 2048), (17, 4096), (100, 6144), (1000, 2048), (148 * 16 + 3, 2048), (9, 768)],
    oracle.Q8_0: [(1, 32), (7, 256), (17, 1024), (100, 4096), (1000, 2048), (148 * 16 + 3, 512), (9, 96)],
}


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("fmt,name", FMTS)
@pytest.mark.parametrize("M", [1, 2, 3, 4, 5, 8])
def test_gemv_matches_oracle(fmt, name, M, path, cpu_oracle):
    set_path(path)
    for N, K in SHAPES[fmt]:
        Wh = synth.make_blocks(fmt, N, K, seed=N * 7 + K)
        Xh = synth.make_activations(M, K, seed=N + K + M)
        want = cpu_oracle.matmul(fmt, Wh, Xh, threads=8)
        got = ops.gemv(fmt, dev(Wh), dev(Xh), N)
        assert got.dtype == torch.float32
        e = oracle.rel_l2(host_f32(got), want)
        assert e < REL_L2, f"N={N} K={K} M={M} rel_l2={e}"


@pytest.mark.parametrize("fmt,name", FMTS)
@pytest.mark.parametrize("M", [3, 4, 5, 7, 8])
def test_gemv_long_rows_several_activation_rows(fmt, name, M, cpu_oracle):
    """K = 14336 (down_proj): eight activation rows do not fit beside the weight ring, so the
    automatic route runs two passes of up to four rows; four rows take the warp-MMA kernel."""
    N, K = 40, 14336
    Wh = synth.make_blocks(fmt, N, K, seed=11)
    Xh = synth.make_activations(M, K, seed=M)
    bias = np.linspace(-1.0, 1.0, N).astype(np.float32)
    want = cpu_oracle.matmul(fmt, Wh, Xh, threads=8) + bias[None, :]
    got = ops.gemv(fmt, dev(Wh), dev(Xh), N, bias=dev(bias))
    e = oracle.rel_l2(host_f32(got), want)
    assert e < REL_L2, f"M={M} rel_l2={e}"
    assert ops.device_status() == 0


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("fmt,name", FMTS)
@pytest.mark.parametrize("xdt,ydt", [("f16", "f16"), ("bf16", "f32"), ("f32", "bf16"), ("bf16", "bf16"), ("f16", "f32")])
def test_gemv_dtypes_and_bias(fmt, name, xdt, ydt, path, cpu_oracle):
    set_path(path)
    N, K, M = 333, 4096 if fmt != oracle.Q6_K else 2048, 3
    Wh = synth.make_blocks(fmt, N, K, seed=21)
    xt, xr = as_dtype_np(synth.make_activations(M, K, seed=22), xdt)
    bt, br = as_dtype_np(synth.make_activations(1, N, seed=23)[0], xdt)
    want = cpu_oracle.matmul(fmt, Wh, xr, bias=br, threads=8)
    got = ops.gemv(fmt, dev(Wh), xt.cuda(), N, bias=bt.cuda(), out_dtype=TORCH_DT[ydt])
    assert got.dtype == TORCH_DT[ydt]
    # the output rounding of a 16-bit Y is part of the contract: allow its half-ulp on top
    tol = REL_L2 + (2.0 ** -9 if ydt == "bf16" else 2.0 ** -12 if ydt == "f16" else 0.0)
    assert oracle.rel_l2(host_f32(got), want) < tol


@pytest.mark.parametrize("fmt,name", FMTS)
def test_three_kernels_agree(fmt, name):
    """Three independent kernels on the same inputs: plain-load FP32, warp-MMA streaming
    (FP16 activations; hi+lo halves when they fit in shared memory, which M=8 at this K
    does not, so one FP16 rounding of x: about 2e-4) and integer-dot streaming
    (int16 fixed-point activations per 128-element group: about 7e-5)."""
    N, K = 2500, 4096 if fmt != oracle.Q6_K else 6144
    W = dev(synth.make_blocks(fmt, N, K, seed=31))
    for M, path, tol in ((8, 2, 5e-4), (4, 3, 2e-4), (1, 3, 2e-4), (2, 2, 1e-5)):
        X = dev(synth.make_activations(M, K, seed=32 + M))
        ops.set_option("gemv_path", 1)
        a = ops.gemv(fmt, W, X, N)
        ops.set_option("gemv_path", path)
        b = ops.gemv(fmt, W, X, N)
        e = oracle.rel_l2(host_f32(b), host_f32(a))
        assert e < tol, f"M={M} path={path}: {e}"


def test_integer_dot_kernel_is_robust_to_outliers(cpu_oracle):
    """Activations with a few huge entries: per-group fixed-point scaling keeps the
    error inside the bound (a per-row scale would not)."""
    fmt, N, K = oracle.Q4_K, 512, 4096
    Wh = synth.make_blocks(fmt, N, K, seed=51)
    Xh = synth.make_activations(2, K, seed=52)
    Xh[0, 7] = 900.0
    Xh[0, 2049] = -350.0
    Xh[1, 4000] = 2.5e4
    Xh[1, 128:256] = 0.0
    want = cpu_oracle.matmul(fmt, Wh, Xh, threads=8)
    ops.set_option("gemv_path", 3)
    got = host_f32(ops.gemv(fmt, dev(Wh), dev(Xh), N))
    assert oracle.rel_l2(got, want) < REL_L2


def test_gemv_is_deterministic_and_linear():
    fmt, N, K = oracle.Q4_K, 4096, 4096
    W = dev(synth.make_blocks(fmt, N, K, seed=41))
    x1 = dev(synth.make_activations(1, K, seed=42))
    x2 = dev(synth.make_activations(1, K, seed=43))
    a = ops.gemv(fmt, W, x1, N)
    assert torch.equal(a, ops.gemv(fmt, W, x1, N))
    s = ops.gemv(fmt, W, x1 + x2, N)
    assert oracle.rel_l2(host_f32(s), host_f32(a + ops.gemv(fmt, W, x2, N))) < 1e-3
    # stacked rows give the same answers as single rows
    both = ops.gemv(fmt, W, torch.cat([x1, x2]), N)
    assert oracle.rel_l2(host_f32(both[0]), host_f32(a[0])) < 1e-5


# ---------------------------------------------------------------- benchmark configurations at full size

def test_config0_q4k_4096(cpu_oracle):
    fmt, N, K = oracle.Q4_K, 4096, 4096
    Wh = synth.make_blocks(fmt, N, K, seed=0)
    Xh = synth.make_activations(1, K, seed=0)
    want, want64 = cpu_oracle.matmul(fmt, Wh, Xh, threads=8, want_f64=True)
    got = host_f32(ops.gemv(fmt, dev(Wh), dev(Xh), N))
    assert oracle.rel_l2(got, want) < REL_L2
    assert oracle.rel_l2(got, want64) < REL_L2


def test_config1_llama_layer_set(cpu_oracle):
    for i, (lname, fmt, N, K) in enumerate(synth.LLAMA3_8B_LAYER_SET):
        Wh = synth.make_blocks(fmt, N, K, seed=100 + i)
        Xh = synth.make_activations(1, K, seed=100 + i)
        want = cpu_oracle.matmul(fmt, Wh, Xh, threads=8)
        got = host_f32(ops.gemv(fmt, dev(Wh), dev(Xh), N))
        e = oracle.rel_l2(got, want)
        assert e < REL_L2, f"{lname}: {e}"


@pytest.mark.parametrize("M", [1, 2, 4, 8])
def test_config2_q8_0_small_batch(M, cpu_oracle):
    fmt, N, K = oracle.Q8_0, 14336, 4096
    Wh = synth.make_blocks(fmt, N, K, seed=2)
    Xh = synth.make_activations(M, K, seed=2)
    want = cpu_oracle.matmul(fmt, Wh, Xh, threads=8)
    got = host_f32(ops.linear(fmt, dev(Wh), dev(Xh), N))
    assert oracle.rel_l2(got, want) < REL_L2


# ---------------------------------------------------------------- prefill GEMM (tensor cores)

@pytest.mark.parametrize("fmt,name", FMTS)
@pytest.mark.parametrize("M,N,K", [(9, 64, 256), (16, 128, 512), (33, 200, 1024), (100, 1000, 2048), (256, 384, 512),
                                   (300, 130, 768), (512, 256, 4096), (700, 77, 512)])
def test_gemm_matches_oracle(fmt, name, M, N, K, cpu_oracle):
    Wh = synth.make_blocks(fmt, N, K, seed=M + N + K)
    Xh = synth.make_activations(M, K, seed=M * 3 + 1)
    bh = synth.make_activations(1, N, seed=5)[0]
    want = cpu_oracle.matmul(fmt, Wh, Xh, bias=bh, threads=8)
    ops.tc_calls_consume(fmt)
    got = ops.gemm(fmt, dev(Wh), dev(Xh), N, bias=dev(bh))
    assert ops.tc_calls_consume(fmt) >= 1  # the tensor-core kernel ran, not the GEMV passes
    assert got.dtype == torch.float32 and tuple(got.shape) == (M, N)
    e = oracle.rel_l2(host_f32(got), want)
    assert e < REL_L2, f"rel_l2={e}"
    # 16-bit activations and outputs
    xt, xr = as_dtype_np(Xh, "bf16")
    want16 = cpu_oracle.matmul(fmt, Wh, xr, threads=8)
    got16 = ops.gemm(fmt, dev(Wh), xt.cuda(), N, out_dtype=torch.float16)
    assert oracle.rel_l2(host_f32(got16), want16) < REL_L2 + 2.0 ** -12


def test_gemm_and_gemv_agree_on_shared_rows():
    """tests/test_quant_prefill_parity.cpp: the prefill path against per-token decode GEMVs."""
    fmt, N, K, M = oracle.Q4_K, 512, 2048, 24
    W = dev(synth.make_blocks(fmt, N, K, seed=61))
    X = dev(synth.make_activations(M, K, seed=62))
    Y = ops.gemm(fmt, W, X, N)
    for m0 in range(0, M, 8):
        y = ops.gemv(fmt, W, X[m0:m0 + 8].contiguous(), N)
        assert oracle.rel_l2(host_f32(Y[m0:m0 + 8]), host_f32(y)) < 1e-3


def test_gemm_workspace_contract():
    from brotensor_b200 import B200QError, _capi
    fmt, N, K, M = oracle.Q4_K, 128, 512, 32
    L = _capi.lib()
    need = L.b200q_gemm_workspace_bytes(fmt, _capi.F32, M, N, K)
    assert need == (K // 64) * 32 * 128
    assert L.b200q_gemm_workspace_bytes(fmt, _capi.F32, 4, N, K) == 0  # decode sizes need none
    W = dev(synth.make_blocks(fmt, N, K, seed=1))
    X = dev(synth.make_activations(M, K, seed=1))
    with pytest.raises(B200QError) as ei:
        ops.gemm(fmt, W, X, N, ws=torch.empty(need - 256, dtype=torch.uint8, device="cuda"))
    assert ei.value.status == _capi.ERR_WORKSPACE


def test_config3_q4k_prefill_512(cpu_oracle):
    """Config 3 at full size: 512 tokens x 14336 x 4096; a strided subset of the output
    columns is checked against the oracle, all of them through linearity in X."""
    fmt, N, K, M = oracle.Q4_K, 14336, 4096, 512
    Wh = synth.make_blocks(fmt, N, K, seed=3)
    Xh = synth.make_activations(M, K, seed=3)
    W, X = dev(Wh), dev(Xh)
    Y = ops.gemm(fmt, W, X, N)
    rows = np.arange(5, N, 97)
    Wsub = Wh.reshape(N, -1)[rows].reshape(-1)
    want = cpu_oracle.matmul(fmt, Wsub, Xh, threads=16)
    assert oracle.rel_l2(host_f32(Y[:, torch.from_numpy(rows).cuda()]), want) < REL_L2
    Yb = ops.gemm(fmt, W, X.bfloat16(), N)
    assert oracle.rel_l2(host_f32(Yb), host_f32(Y)) < 6e-3  # bf16 rounding of x alone is 2^-9 / sqrt(3)
    Y2 = ops.gemm(fmt, W, X * 2.0, N)
    assert oracle.rel_l2(host_f32(Y2), 2.0 * host_f32(Y)) < 1e-6


# ---------------------------------------------------------------- error behaviour

def test_bad_arguments_raise():
    from brotensor_b200 import B200QError
    W = dev(synth.make_blocks(oracle.Q4_K, 4, 256, seed=1))
    x = dev(synth.make_activations(9, 256, seed=1))
    with pytest.raises(B200QError):
        ops.gemv(oracle.Q4_K, W, x, 4)  # M > 8
    with pytest.raises(ValueError):
        ops.gemv(oracle.Q4_K, W, x[:1, :128].contiguous(), 4)  # K not a block multiple
    assert ops.gemv(oracle.Q4_K, W[:0], x[:1], 0).shape == (1, 0)


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,N,K,M", [(synth.Q4_K, 256, 256, 16), (synth.Q4_K, 384, 512, 48), (synth.Q4_K, 1024, 1024, 272),
                                       (synth.Q4_K, 1000, 768, 700), (synth.Q6_K, 256, 512, 33), (synth.Q8_0, 384, 512, 130),
                                       (synth.Q4_K, 2048, 2048, 512)])
def test_gemm_cta_pair_equals_single_cta(fmt, N, K, M, cpu_oracle):
    """The CTA-pair kernel (cta_group::2, two alternating issuers) queues its MMAs in the same
    k order as the one-CTA kernel, so the two agree bit for bit; both agree with the oracle."""
    import torch
    import oracle
    Wh = synth.make_blocks(fmt, N, K, seed=N + M)
    xh = synth.make_activations(M, K, seed=M)
    W, X = torch.from_numpy(Wh).cuda(), torch.from_numpy(xh).cuda()
    try:
        ops.set_option("gemm_split", 0)  # a split K adds the partial sums in another order
        ops.set_option("gemm_pair", 0)
        y0 = ops.gemm(fmt, W, X, N)
        ops.set_option("gemm_pair", 1)
        y1 = ops.gemm(fmt, W, X, N)
        y2 = ops.gemm(fmt, W, X, N)
    finally:
        ops.set_option("gemm_pair", -1)
        ops.set_option("gemm_split", 1)
    torch.cuda.synchronize()
    assert torch.equal(y1, y2)  # same on every run
    assert torch.equal(y0, y1)
    assert oracle.rel_l2(y1.cpu().numpy(), cpu_oracle.matmul(fmt, Wh, xh, threads=8)) < 2e-3
    assert ops.device_status() == 0


@pytest.mark.gpu
def test_gemm_seeded_shapes_against_the_oracle(cpu_oracle):
    """Two dozen seeded shapes across the prefill routes (tcgen05 pairs with and without a split K, GEMV passes for
    small M, odd row counts, several passes of 512 tokens, every format the tensor-core kernel takes, bias on or
    off, FP32 / FP16 / BF16 activations): each within the prefill bound of the oracle and the same on a second run."""
    import torch
    import oracle
    rng = np.random.default_rng(20240611)
    fmts = [synth.Q4_K, synth.Q6_K, synth.Q8_0]
    for case in range(24):
        fmt = fmts[case % 3]
        N = int(rng.choice([1, 7, 64, 100, 129, 255, 256, 300, 511, 1000, 1028, 2052, 4096]))
        K = 256 * int(rng.choice([1, 2, 3, 4, 8, 12, 16, 32]))
        M = int(rng.choice([9, 12, 16, 17, 31, 64, 100, 257, 513, 600]))
        if N * K * M > 1.5e9:
            M = 17
        dt = [torch.float32, torch.float16, torch.bfloat16][int(rng.integers(0, 3))]
        with_bias = bool(rng.integers(0, 2))
        Wh = synth.make_blocks(fmt, N, K, seed=1000 + case)
        xh = synth.make_activations(M, K, seed=2000 + case)
        bh = synth.make_activations(1, N, seed=3000 + case).reshape(-1)
        W, X = torch.from_numpy(Wh).cuda(), torch.from_numpy(xh).cuda().to(dt)
        b = torch.from_numpy(bh).cuda().to(dt) if with_bias else None
        y1 = ops.gemm(fmt, W, X, N, bias=b)
        y2 = ops.gemm(fmt, W, X, N, bias=b)
        assert torch.equal(y1, y2), (case, fmt, N, K, M)
        want = cpu_oracle.matmul(fmt, Wh, X.float().cpu().numpy(), bias=b.float().cpu().numpy() if with_bias else None, threads=16)
        r = oracle.rel_l2(y1.float().cpu().numpy(), want)
        assert r < 2e-3, (case, fmt, N, K, M, str(dt), with_bias, r)
    assert ops.device_status() == 0


@pytest.mark.gpu
def test_gemm_split_k_needs_aligned_outputs():
    """The reduction after a split K moves four outputs at a time; a result or FP32 bias that is only aligned to its
    element size gets the unsplit kernel (bit for bit), not a misaligned access."""
    import torch
    fmt, N, K, M = synth.Q4_K, 1024, 4096, 40
    W = torch.from_numpy(synth.make_blocks(fmt, N, K, seed=9)).cuda()
    X = torch.from_numpy(synth.make_activations(M, K, seed=9)).cuda()
    b = torch.from_numpy(synth.make_activations(1, N + 1, seed=5).reshape(-1)).cuda()
    try:
        ops.set_option("gemm_split", 0)
        y0 = ops.gemm(fmt, W, X, N, bias=b[1:].clone())
    finally:
        ops.set_option("gemm_split", 1)
    big = torch.zeros(M * N + 1, dtype=torch.float32, device="cuda")
    y_off = big[1:].view(M, N)                      # 4-byte aligned only
    ops.gemm(fmt, W, X, N, bias=b[1:].clone(), out=y_off)
    assert torch.equal(y_off, y0)
    y_b = ops.gemm(fmt, W, X, N, bias=b[1:])        # bias 4-byte aligned only
    assert torch.equal(y_b, y0)
    assert ops.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,N,K,M", [(synth.Q4_K, 600, 4096, 16), (synth.Q8_0, 333, 2048, 9), (synth.Q6_K, 8192, 2048, 12),
                                       (synth.Q4_K, 14336, 4096, 13)])
def test_gemm_of_nine_to_sixteen_rows(fmt, N, K, M, cpu_oracle):
    """9..16 rows of these shapes run as two passes of the small-batch GEMV instead of the tcgen05 GEMM (the faster
    form there): within the GEMV's bound of the oracle, close to the tensor-core GEMM, counted as a tensor-core
    call, bias and 16-bit types included, no workspace needed."""
    import torch
    import oracle
    Wh = synth.make_blocks(fmt, N, K, seed=N + M)
    xh = synth.make_activations(M, K, seed=M)
    bh = synth.make_activations(1, N, seed=5).reshape(-1)
    W, X, b = torch.from_numpy(Wh).cuda(), torch.from_numpy(xh).cuda(), torch.from_numpy(bh).cuda()
    try:
        ops.set_option("gemm_path", 2)
        y_tc = ops.gemm(fmt, W, X, N, bias=b)
        ops.set_option("gemm_path", 0)
        ops.tc_calls_consume(fmt)
        y = ops.gemm(fmt, W, X, N, bias=b)
        assert ops.tc_calls_consume(fmt) == 1
        yh = ops.gemm(fmt, W, X.half(), N, bias=b.half(), out_dtype=torch.float16)
    finally:
        ops.set_option("gemm_path", 0)
    rows = np.arange(0, N, max(1, N // 500))
    want = cpu_oracle.matmul(fmt, Wh.reshape(N, -1)[rows].reshape(-1), xh, threads=16) + bh[None, rows]
    cols = torch.from_numpy(rows).cuda()
    assert oracle.rel_l2(y[:, cols].cpu().numpy(), want) < 2e-3
    assert oracle.rel_l2(yh[:, cols].float().cpu().numpy(), want) < 2e-3
    assert oracle.rel_l2(y.cpu().numpy(), y_tc.cpu().numpy()) < 2e-3  # FP16 operands there, fixed-point activations here
    for m0 in range(0, M, 8):
        assert torch.equal(y[m0:m0 + 8], ops.gemv(fmt, W, X[m0:m0 + 8].contiguous(), N, bias=b))
    assert ops.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,N,K,M", [(synth.Q4_K, 1024, 1024, 272), (synth.Q4_K, 4096, 4096, 512), (synth.Q6_K, 4096, 14336, 200),
                                       (synth.Q8_0, 1000, 4096, 64), (synth.Q4_K, 2048, 2048, 600), (synth.Q6_K, 300, 8192, 17)])
def test_gemm_split_k(fmt, N, K, M, cpu_oracle):
    """Few row tiles and long rows: the k-blocks of a row tile are split over several CTA pairs and the partial
    sums added in a fixed order by a second kernel. Same result on every run, equal to the unsplit kernel up
    to the order of the FP32 additions, within the prefill bound of the oracle; bias and FP16 output included;
    more than one pass of 512 tokens reuses the partial-sum buffer."""
    import torch
    import oracle
    from brotensor_b200 import _capi
    Wh = synth.make_blocks(fmt, N, K, seed=N + M)
    xh = synth.make_activations(M, K, seed=M)
    bh = synth.make_activations(1, N, seed=5).reshape(-1)
    W, X, b = torch.from_numpy(Wh).cuda(), torch.from_numpy(xh).cuda(), torch.from_numpy(bh).cuda()
    L = _capi.lib()
    try:
        ops.set_option("gemm_split", 0)
        need0 = L.b200q_gemm_workspace_bytes(fmt, _capi.F32, M, N, K)
        y0 = ops.gemm(fmt, W, X, N, bias=b)
        ops.set_option("gemm_split", 1)
        need1 = L.b200q_gemm_workspace_bytes(fmt, _capi.F32, M, N, K)
        y1 = ops.gemm(fmt, W, X, N, bias=b)
        y2 = ops.gemm(fmt, W, X, N, bias=b)
        yh = ops.gemm(fmt, W, X.half(), N, bias=b.half(), out_dtype=torch.float16)
        ysmall = ops.gemm(fmt, W, X, N, bias=b, ws=torch.empty(need0, dtype=torch.uint8, device="cuda"))  # room for the image only
    finally:
        ops.set_option("gemm_split", 1)
    torch.cuda.synchronize()
    assert need1 > need0 and (need1 - need0) % (min(M, 512) * N * 4) == 0  # the partial sums of 2..8 splits
    assert torch.equal(y1, y2)
    assert torch.equal(ysmall, y0)  # given no room for partial sums the call runs unsplit
    r = oracle.rel_l2(y1.cpu().numpy(), y0.cpu().numpy())
    assert r < 1e-4, r  # the order of the FP32 additions alone
    want = cpu_oracle.matmul(fmt, Wh, xh, threads=16) + bh[None, :]
    assert oracle.rel_l2(y1.cpu().numpy(), want) < 2e-3
    assert oracle.rel_l2(yh.float().cpu().numpy(), want) < 4e-3
    assert ops.device_status() == 0



@pytest.mark.gpu
@pytest.mark.parametrize("fmt,K,Ns", [(synth.Q4_K, 4096, [4096, 1024, 1024]), (synth.Q4_K, 512, [100, 7, 33, 16]),
                                      (synth.Q6_K, 2048, [256, 300]), (synth.Q8_0, 256, [48, 1000]), (synth.Q4_K, 4096, [14336, 14336])])
def test_grouped_gemv_equals_separate_launches(fmt, K, Ns, cpu_oracle):
    """Several matrices against one activation vector in one launch: bit-identical to one launch each."""
    Whs = [synth.make_blocks(fmt, N, K, seed=10 + i) for i, N in enumerate(Ns)]
    Ws = [torch.from_numpy(w).cuda() for w in Whs]
    xh = synth.make_activations(1, K, seed=4)
    x = torch.from_numpy(xh).cuda()
    biases = [torch.from_numpy(synth.make_activations(1, N, seed=20 + i)).cuda().view(-1) if i % 2 == 0 else None
              for i, N in enumerate(Ns)]
    outs = ops.gemv_multi(fmt, Ws, x, Ns, biases=biases)
    torch.cuda.synchronize()
    for W, Wh, N, b, y in zip(Ws, Whs, Ns, biases, outs):
        ref = ops.gemv(fmt, W, x, N, bias=b)
        assert torch.equal(y, ref)
        if N <= 4096:
            want = cpu_oracle.matmul(fmt, Wh, xh, threads=8)
            if b is not None:
                want = want + b.cpu().numpy()[None, :]
            assert oracle.rel_l2(y.cpu().numpy(), want) < 2e-3
    assert ops.device_status() == 0


@pytest.mark.gpu
def test_grouped_gemv_argument_checks():
    fmt, K = synth.Q4_K, 256
    W = torch.from_numpy(synth.make_blocks(fmt, 16, K, seed=1)).cuda()
    x = torch.zeros(K, device="cuda")
    with pytest.raises(Exception):
        ops.gemv_multi(fmt, [W] * 5, x, [16] * 5)       # more than four matrices


# ---- device-side repack (Q6_K regrouped by field in runs of eight blocks) ------------------------

def _q6_runs_on_host(raw: np.ndarray) -> np.ndarray:
    """The regrouped layout restated with numpy: per run of eight 210-byte blocks,
    ql[8][128] | qh[8][64] | scales[8][16] | d[8][2]."""
    b = raw.reshape(-1, 8, 210)
    return np.concatenate([b[:, :, :128].reshape(-1, 1024), b[:, :, 128:192].reshape(-1, 512),
                           b[:, :, 192:208].reshape(-1, 128), b[:, :, 208:210].reshape(-1, 16)], axis=1).reshape(-1)


@pytest.mark.parametrize("N,K", [(1, 2048), (37, 4096), (300, 14336)])
def test_repack_q6k_is_a_permutation_and_round_trips(N, K):
    raw = synth.make_blocks(synth.Q6_K, N, K, seed=N + K)
    assert ops.repacked_fmt(synth.Q6_K, K) == synth.Q6_K_R8
    packed = ops.repack(synth.Q6_K, dev(raw), N, K)
    assert np.array_equal(packed.cpu().numpy(), _q6_runs_on_host(raw))
    back = ops.unpack(synth.Q6_K, packed, N, K)
    assert np.array_equal(back.cpu().numpy(), raw)
    # in place, both directions
    w = dev(raw).clone()
    ops.repack(synth.Q6_K, w, N, K, inplace=True)
    assert np.array_equal(w.cpu().numpy(), _q6_runs_on_host(raw))
    ops.unpack(synth.Q6_K, w, N, K, inplace=True)
    assert np.array_equal(w.cpu().numpy(), raw)


def test_repack_without_a_regrouped_form_copies():
    for fmt, K in ((synth.Q4_K, 1024), (synth.Q8_0, 256), (synth.Q6_K, 768)):
        assert ops.repacked_fmt(fmt, K) == fmt
        raw = synth.make_blocks(fmt, 9, K, seed=3)
        assert np.array_equal(ops.repack(fmt, dev(raw), 9, K).cpu().numpy(), raw)
        assert np.array_equal(ops.unpack(fmt, dev(raw), 9, K).cpu().numpy(), raw)


@pytest.mark.parametrize("N,K", [(40, 2048), (1000, 4096), (148 * 16 + 3, 2048), (64, 14336)])
def test_repacked_q6k_gives_the_same_bits(N, K, cpu_oracle):
    """Every op on the regrouped layout equals the op on the raw layout bit for bit: decode,
    decode GEMV (1..8 rows), sharded-form arguments aside, and the prefill GEMM."""
    raw = synth.make_blocks(synth.Q6_K, N, K, seed=N * 3 + K)
    Wr = dev(raw)
    Wp = ops.repack(synth.Q6_K, Wr, N, K)
    for dt in (torch.float16, torch.float32, torch.bfloat16):
        assert torch.equal(ops.dequant(synth.Q6_K_R8, Wp, N, K, out_dtype=dt), ops.dequant(synth.Q6_K, Wr, N, K, out_dtype=dt))
    for M in (1, 2, 4, 8):
        X = dev(synth.make_activations(M, K, seed=M))
        got = ops.gemv(synth.Q6_K_R8, Wp, X, N)
        want = cpu_oracle.matmul(synth.Q6_K, raw, X.cpu().numpy(), threads=8)
        assert oracle.rel_l2(host_f32(got), want) < REL_L2
        if M <= 2:  # the same kernel and the same order of arithmetic on both layouts
            assert torch.equal(got, ops.gemv(synth.Q6_K, Wr, X, N))
    X = dev(synth.make_activations(48, K, seed=7))
    assert torch.equal(ops.gemm(synth.Q6_K_R8, Wp, X, N), ops.gemm(synth.Q6_K, Wr, X, N))
    assert ops.device_status() == 0


# ---- gate / up projection with the SwiGLU gate in the epilogue -----------------------------------

@pytest.mark.parametrize("fmt,N,K", [(synth.Q4_K, 14336, 4096), (synth.Q4_K, 100, 512), (synth.Q4_K, 7, 256), (synth.Q6_K, 333, 2048),
                                     (synth.Q8_0, 1000, 1024), (synth.Q4_K, 148 * 8 + 3, 1024)])
def test_gemv_swiglu_equals_two_gemvs_and_the_gate(fmt, N, K, cpu_oracle):
    """silu(gate . x) * (up . x) from one launch: the two dot products are the separate launches'
    bits, the gate follows brotensor's swiglu_forward (v / (1 + exp(-v)) * u)."""
    Wg, Wu = synth.make_blocks(fmt, N, K, seed=N + 1), synth.make_blocks(fmt, N, K, seed=N + 2)
    x = synth.make_activations(1, K, seed=K)
    xd = dev(x)
    got = host_f32(ops.gemv_swiglu(fmt, dev(Wg), dev(Wu), xd, N))
    g = host_f32(ops.gemv(fmt, dev(Wg), xd, N)).astype(np.float64)
    u = host_f32(ops.gemv(fmt, dev(Wu), xd, N)).astype(np.float64)
    same_sums = g / (1.0 + np.exp(-g)) * u
    assert np.allclose(got, same_sums, rtol=2e-6, atol=1e-30)
    wg, wu = cpu_oracle.matmul(fmt, Wg, x, threads=8).astype(np.float64), cpu_oracle.matmul(fmt, Wu, x, threads=8).astype(np.float64)
    assert oracle.rel_l2(got, (wg / (1.0 + np.exp(-wg)) * wu).astype(np.float32)) < REL_L2
    h = host_f32(ops.gemv_swiglu(fmt, dev(Wg), dev(Wu), xd.half(), N, out_dtype=torch.float16))
    assert oracle.rel_l2(h, got) < 2e-3
    assert ops.device_status() == 0


# ---- RMSNorm folded into the GEMV's activation staging --------------------------------------------

@pytest.mark.parametrize("fmt,K,Ns", [(synth.Q4_K, 4096, [4096, 1024, 1024]), (synth.Q4_K, 4096, [14336, 14336]), (synth.Q6_K, 2048, [50]),
                                      (synth.Q8_0, 1024, [100, 7]), (synth.Q6_K, 14336, [64])])
@pytest.mark.parametrize("xdt", [torch.float32, torch.float16])
def test_rmsnorm_folded_into_grouped_gemv(fmt, K, Ns, xdt, cpu_oracle):
    """y_s = W_s (x * gamma * rsqrt(mean x^2 + eps)): brotensor's rms_norm_forward followed by its
    GEMVs, in one launch; compared with the oracle on the host-normalised vector."""
    eps = 1e-5
    x = (synth.make_activations(1, K, seed=K + len(Ns)) * 3.0).astype(np.float32)
    gamma = (1.0 + 0.1 * synth.make_activations(1, K, seed=7)).astype(np.float32)
    xd, gd = dev(x).to(xdt).view(-1), dev(gamma).to(xdt).view(-1)
    xh, gh = xd.float().cpu().numpy().astype(np.float64), gd.float().cpu().numpy().astype(np.float64)
    xn = (xh * gh / np.sqrt(np.mean(xh * xh) + eps)).astype(np.float32).reshape(1, K)
    Ws = [synth.make_blocks(fmt, N, K, seed=N + i) for i, N in enumerate(Ns)]
    got = ops.gemv_multi_rmsnorm(fmt, [dev(W) for W in Ws], xd, gd, eps, Ns)
    for W, N, y in zip(Ws, Ns, got):
        want = cpu_oracle.matmul(fmt, W, xn, threads=8)
        assert oracle.rel_l2(host_f32(y), want) < REL_L2, f"N={N}"
    # the same launch without the fold on the host-normalised vector: equal up to the rounding of xn
    plain = [ops.gemv(fmt, dev(W), dev(xn), N) for W, N in zip(Ws, Ns)]
    for a, b in zip(got, plain):
        assert oracle.rel_l2(host_f32(a), host_f32(b)) < 2e-4
    assert ops.device_status() == 0

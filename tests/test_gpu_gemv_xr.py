"""The activation-resident Q4_K / Q6_K decode GEMV (csrc/gemv_xr.cu) against the CPU oracle and against the
16-row-tile kernel it stands in for: same arithmetic, so the two must agree bit for bit, for every
element type, with and without bias, on ragged row counts (odd, fewer pairs than warps, fewer than
SMs) and short rows (K < 4096 leaves lanes without a group)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

import oracle
from brotensor_b200 import synth

SHAPES = [(1, 256), (2, 256), (3, 512), (31, 768), (17, 1024), (295, 2048), (600, 4096), (1025, 4096), (4097, 2048),
          (333, 3840), (4736, 4096), (14336, 4096)]


@pytest.fixture
def xr_option():
    from brotensor_b200 import ops
    yield ops
    ops.set_option("gemv_xr", 1)
    ops.set_option("pdl", 0)


Q6_SHAPES = [(1, 2048), (2, 4096), (31, 2048), (600, 4096), (1025, 4096), (4736, 4096), (16032, 4096)]


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,N,K", [(synth.Q4_K, n, k) for n, k in SHAPES] + [(synth.Q6_K, n, k) for n, k in Q6_SHAPES])
def test_xr_matches_oracle_and_tile_kernel_bit_for_bit(fmt, N, K, xr_option):
    ops = xr_option
    cpu = oracle.cpu()
    Wh = synth.make_blocks(fmt, N, K, seed=N + K)
    Xh = synth.make_activations(1, K, seed=K)
    bh = synth.make_activations(1, N, seed=7).reshape(-1)
    W, X, b = torch.from_numpy(Wh).cuda(), torch.from_numpy(Xh).cuda(), torch.from_numpy(bh).cuda()
    want = cpu.matmul(fmt, Wh, Xh, threads=8)
    for dt in (torch.float32, torch.float16, torch.bfloat16):
        for bias in (None, b.to(dt)):
            got = {}
            for xr in (0, 2):
                ops.set_option("gemv_xr", xr)
                got[xr] = ops.gemv(fmt, W, X.to(dt), N, bias=bias, out_dtype=dt).float().cpu().numpy()
            assert np.array_equal(got[0], got[2]), f"{dt} bias={bias is not None}: kernels differ"
    ops.set_option("gemv_xr", 2)
    y = ops.gemv(fmt, W, X, N).cpu().numpy()
    assert oracle.rel_l2(y, want) < 2e-3  # tolerance of the decode GEMV against the FP32 oracle
    assert ops.device_status() == 0


@pytest.mark.gpu
def test_xr_back_to_back_under_dependent_launch(xr_option):
    """A captured chain of launches (each may start its weight copies while its predecessor drains) gives
    the single launch's bits, on rotating weights."""
    ops = xr_option
    ops.set_option("pdl", 1)
    ops.set_option("gemv_xr", 2)
    N, K, R = 14336, 4096, 3
    Ws = [torch.from_numpy(synth.make_blocks(synth.Q4_K, N, K, seed=50 + r)).cuda() for r in range(R)]
    X = torch.from_numpy(synth.make_activations(1, K, seed=9)).cuda()
    single = [ops.gemv(synth.Q4_K, W, X, N).clone() for W in Ws]
    outs = [torch.empty((1, N), dtype=torch.float32, device="cuda") for _ in range(12)]
    g, st = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.graph(g, stream=st):
        for i, y in enumerate(outs):
            ops.gemv(synth.Q4_K, Ws[i % R], X, N, out=y)
    for _ in range(5):
        g.replay()
    torch.cuda.synchronize()
    for i, y in enumerate(outs):
        assert torch.equal(y, single[i % R])
    assert ops.device_status() == 0

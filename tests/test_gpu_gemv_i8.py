"""The integer tensor-core small-batch GEMV (csrc/gemv_i8.cu: Q8_0 and Q4_K, 2..8 activation rows, K = 2048
or 4096) against the CPU oracle's FP32 result (rel-L2 <= 2e-3, the decode GEMV's bound) and against the
kernels it stands in for; ragged row counts (fewer rows than a 16-row tile, a tail tile, fewer tiles than
SMs), every element type, with and without bias, and a captured chain under dependent launch."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

import oracle
from brotensor_b200 import synth


@pytest.fixture
def ops_i8():
    from brotensor_b200 import ops
    yield ops
    ops.set_option("gemv_i8", 1)
    ops.set_option("pdl", 0)


@pytest.mark.gpu
@pytest.mark.parametrize("N,K", [(1, 2048), (15, 4096), (16, 2048), (17, 4096), (600, 4096), (2369, 2048), (14336, 4096)])
@pytest.mark.parametrize("M", [2, 3, 5, 8])
@pytest.mark.parametrize("fmt", [synth.Q8_0, synth.Q4_K])
def test_i8_matches_oracle_and_the_other_kernels(fmt, N, K, M, ops_i8):
    ops = ops_i8
    cpu = oracle.cpu()
    Wh = synth.make_blocks(fmt, N, K, seed=N + K + M)
    Xh = synth.make_activations(M, K, seed=K + M)
    bh = synth.make_activations(1, N, seed=3).reshape(-1)
    W, X, b = torch.from_numpy(Wh).cuda(), torch.from_numpy(Xh).cuda(), torch.from_numpy(bh).cuda()
    want = cpu.matmul(fmt, Wh, Xh, threads=8)
    ops.set_option("gemv_i8", 2)  # every shape that qualifies, also those another kernel is faster on
    got = ops.gemv(fmt, W, X, N).cpu().numpy()
    assert got.shape == (M, N)
    assert oracle.rel_l2(got, want) < 2e-3
    ops.set_option("gemv_i8", 0)
    other = ops.gemv(fmt, W, X, N).cpu().numpy()
    assert oracle.rel_l2(got, other) < 2e-3
    for dt in (torch.float16, torch.bfloat16):
        ops.set_option("gemv_i8", 2)
        y = ops.gemv(fmt, W, X.to(dt), N, bias=b.to(dt), out_dtype=dt).float().cpu().numpy()
        ref = cpu.matmul(fmt, Wh, X.to(dt).float().cpu().numpy(), bias=b.to(dt).float().cpu().numpy(), threads=8)
        assert oracle.rel_l2(y, ref) < (4e-3 if dt == torch.bfloat16 else 2e-3)  # bf16 output rounding: 2^-9 per element
    assert ops.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", [synth.Q8_0, synth.Q4_K])
def test_i8_reproducible_and_in_a_captured_chain(fmt, ops_i8):
    ops = ops_i8
    ops.set_option("pdl", 1)
    ops.set_option("gemv_i8", 2)
    N, K, M, R = 14336, 4096, 8, 3
    Ws = [torch.from_numpy(synth.make_blocks(fmt, N, K, seed=60 + r)).cuda() for r in range(R)]
    X = torch.from_numpy(synth.make_activations(M, K, seed=9)).cuda()
    single = [ops.gemv(fmt, W, X, N).clone() for W in Ws]
    assert torch.equal(single[0], ops.gemv(fmt, Ws[0], X, N))  # fixed summation order
    outs = [torch.empty((M, N), dtype=torch.float32, device="cuda") for _ in range(9)]
    g, st = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.graph(g, stream=st):
        for i, y in enumerate(outs):
            ops.gemv(fmt, Ws[i % R], X, N, out=y)
    for _ in range(4):
        g.replay()
    torch.cuda.synchronize()
    for i, y in enumerate(outs):
        assert torch.equal(y, single[i % R])
    assert ops.device_status() == 0

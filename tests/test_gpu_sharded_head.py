"""Row-sharded LM head, fused form: the shard GEMV stores its rows into every rank's result
vector and signals arrival in the same kernel (b200q_gemv_shard through the C++ ShardedHead).

One GPU: a single rank exercises the peer-table stores, the arrival words and the
alternating result vectors. Two or more GPUs: real ranks under torchrun (skipped otherwise)."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

from brotensor_b200 import synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,N,K", [(synth.Q6_K, 4096 + 48, 2048), (synth.Q4_K, 1000, 512), (synth.Q8_0, 513, 256)])
def test_single_rank_head_matches_gemv_and_oracle(fmt, N, K, cpu_oracle):
    import torch
    from brotensor_b200 import hostapi, ops
    import oracle
    hostapi.init()
    Wh = synth.make_blocks(fmt, N, K, seed=N)
    w = hostapi.Weight(fmt, Wh, N, K, 0)
    head = hostapi.ShardedHead(w, 0, N, 0, 1)
    Wd = torch.from_numpy(Wh).cuda()
    prev = None
    for call in range(3):
        xh = synth.make_activations(1, K, seed=50 + call)
        x = torch.from_numpy(xh).cuda()
        torch.cuda.synchronize()
        head.run(x.data_ptr(), K, 0)
        got = head.logits()
        assert head.calls() == call + 1
        ref = ops.gemv(fmt, Wd, x, N).cpu().numpy().reshape(-1)
        assert np.array_equal(got, ref), f"call {call}"            # same kernel, same arithmetic
        assert oracle.rel_l2(got, cpu_oracle.matmul(fmt, Wh, xh, threads=4).reshape(-1)) < 2e-3
        if prev is not None:
            assert not np.array_equal(got, prev)
        prev = got
    assert ops.device_status() == 0
    head.close()


@pytest.mark.gpu
def test_lm_head_full_size_against_the_oracle(cpu_oracle):
    """The LM-head configuration at its full size: Q6_K 128256 x 4096, one activation row. The plain
    GEMV and the single-rank sharded head against the CPU oracle's FP32 result, bound rel-L2 2e-3
    (the reference checks its Q6_K GEMV the same way on small shapes, tests/test_q6k_parity.cpp:139-151)."""
    import torch
    from brotensor_b200 import hostapi, ops
    import oracle
    fmt, N, K = synth.Q6_K, 128256, 4096
    Wh = synth.make_blocks(fmt, N, K, seed=4)
    xh = synth.make_activations(1, K, seed=4)
    want = cpu_oracle.matmul(fmt, Wh, xh, threads=os.cpu_count() or 1).reshape(-1)
    Wd = torch.from_numpy(Wh).cuda()
    x = torch.from_numpy(xh).cuda()
    got = ops.gemv(fmt, Wd, x, N).cpu().numpy().reshape(-1)
    assert got.shape == (N,)
    err = oracle.rel_l2(got, want)
    assert err < 2e-3, f"gemv: rel-L2 {err}"
    hostapi.init()
    w = hostapi.Weight.view(fmt, Wd.data_ptr(), N, K, 0)
    head = hostapi.ShardedHead(w, 0, N, 0, 1)
    torch.cuda.synchronize()
    head.run(x.data_ptr(), K, 0)
    logits = head.logits()
    assert np.array_equal(logits, got)  # the same kernel arithmetic
    assert oracle.rel_l2(logits, want) < 2e-3
    assert ops.device_status() == 0
    head.close()


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,N,K", [(synth.Q6_K, 4096 + 48, 2048), (synth.Q4_K, 1000, 512), (synth.Q8_0, 5, 256)])
def test_single_rank_candidate_form(fmt, N, K):
    """Greedy / top-k form: the k largest logits and their rows, largest first, equal values keep the
    lower row (brotensor's rule at temperature 0, include/brotensor/ops/sampling.h:27-28). Checked
    against a sort of the same kernel's full logits, with ties forced by duplicated weight rows."""
    import torch
    from brotensor_b200 import hostapi, ops
    hostapi.init()
    Wh = synth.make_blocks(fmt, N, K, seed=N).reshape(N, -1)
    Wh[N // 2] = Wh[1]          # equal logits at rows 1 and N // 2, whatever the activations
    Wh[N - 1] = Wh[1]
    Wh = np.ascontiguousarray(Wh).reshape(-1)
    w = hostapi.Weight(fmt, Wh, N, K, 0)
    head = hostapi.ShardedHead(w, 0, N, 0, 1)
    Wd = torch.from_numpy(Wh).cuda()
    for call, k in enumerate((1, 3, 8, 1, 8)):
        xh = synth.make_activations(1, K, seed=70 + call)
        if call >= 3:            # make the tied rows the winners
            xh = np.ascontiguousarray(xh)
        x = torch.from_numpy(xh).cuda()
        full = ops.gemv(fmt, Wd, x, N).cpu().numpy().reshape(-1)
        torch.cuda.synchronize()
        head.run_topk(x.data_ptr(), K, k, 0)
        vals, rows = head.top(k)
        kk = min(k, N)
        order = np.lexsort((np.arange(N), -full))[:kk]
        assert np.array_equal(rows[:kk], order.astype(np.int32)), f"call {call}: {rows} vs {order}"
        assert np.array_equal(vals[:kk], full[order])
        if k > N:
            assert np.all(np.isneginf(vals[N:]))
        if call == 2:            # a full forward in between uses the same exchange memory
            head.run(x.data_ptr(), K, 0)
            assert np.array_equal(head.logits(), full)
    # ties among the winners: scale the activations so that the duplicated rows lead
    assert ops.device_status() == 0
    head.close()


@pytest.mark.gpu
def test_candidate_form_argument_checks():
    from brotensor_b200 import hostapi
    hostapi.init()
    fmt, N, K = synth.Q4_K, 64, 256
    w = hostapi.Weight(fmt, synth.make_blocks(fmt, N, K, seed=1), N, K, 0)
    head = hostapi.ShardedHead(w, 0, N, 0, 1)
    for k in (0, 9, -1):
        with pytest.raises(RuntimeError, match="sharded_head"):
            head.run_topk(0, K, k, 0)
    head.close()


@pytest.mark.gpu
def test_head_argument_checks():
    from brotensor_b200 import hostapi
    hostapi.init()
    fmt, N, K = synth.Q4_K, 64, 256
    w = hostapi.Weight(fmt, synth.make_blocks(fmt, N, K, seed=1), N, K, 0)
    with pytest.raises(RuntimeError, match="sharded_head"):
        hostapi.ShardedHead(w, 10, 64, 0, 1)       # rows 10..74 of 64
    with pytest.raises(RuntimeError, match="sharded_head"):
        hostapi.ShardedHead(w, 0, 64, 3, 2)        # rank out of range


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.gpu
def test_two_rank_head_matches_all_gather():
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs")
    world = 2
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "dist_gpu_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0 and "HEAD_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]

"""b200q_gemm_static: the prefill GEMM with its scratch in the library's fixed device array.

Collected last on purpose: it has to pass on its own and after every other test has used
the library (and the shared array's neighbours in device memory)."""
import numpy as np
import pytest

from brotensor_b200 import _capi, synth


def test_static_scratch_limit_is_declared():
    L = _capi.lib()
    cap = L.b200q_gemm_static_max_bytes()
    assert cap == 8 << 20
    # the headline prefill shape fits, with room to spare
    assert 0 < L.b200q_gemm_workspace_bytes(synth.Q4_K, 0, 512, 14336, 4096) <= cap
    # a request beyond the array is refused before any device work (also without a GPU)
    M, K = 2048, 8192
    assert L.b200q_gemm_workspace_bytes(synth.Q4_K, 0, M, 256, K) > cap
    rc = L.b200q_gemm_static(synth.Q4_K, 16, 16, 0, None, 16, 0, M, 256, K, None)
    assert rc == _capi.ERR_WORKSPACE
    msg = L.b200q_last_error().decode()
    assert "gemm_static" in msg and "caller-owned workspace" in msg


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,N,K,M", [(synth.Q4_K, 512, 1024, 96), (synth.Q6_K, 256, 512, 33), (synth.Q8_0, 384, 512, 130),
                                       (synth.Q4_K, 14336, 4096, 512)])
def test_static_matches_workspace_form_twice(fmt, N, K, M):
    import torch
    from brotensor_b200 import ops
    W = torch.from_numpy(synth.make_blocks(fmt, N, K, seed=N + M)).cuda()
    bias = torch.from_numpy(synth.make_activations(1, N, seed=5)).cuda().view(-1)
    outs = []
    # two calls in a row with different activations: the second must not see the first's image
    for call in range(2):
        X = torch.from_numpy(synth.make_activations(M, K, seed=100 + call)).cuda()
        ref = ops.gemm(fmt, W, X, N, bias=bias)
        ops.tc_calls_consume(fmt)
        got = torch.empty_like(ref)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        ops.gemm_static(fmt, W, X, N, bias=bias, out=got)
        torch.cuda.synchronize()
        if call == 1:  # the kernels' code is resident after the first call: the second must not take a byte of device memory
            assert torch.cuda.mem_get_info()[0] == free_before, "gemm_static allocated device memory"
        assert ops.tc_calls_consume(fmt) == 1  # the tensor-core kernel ran, not a fallback
        assert torch.equal(got, ref), f"call {call}: max diff {(got - ref).abs().max().item()}"
        outs.append(got)
    assert not torch.equal(outs[0], outs[1])
    assert ops.device_status() == 0


@pytest.mark.gpu
def test_static_small_m_routes_like_gemm():
    import torch
    from brotensor_b200 import ops
    fmt, N, K, M = synth.Q4_K, 256, 512, 4  # below the tensor-core threshold: no scratch at all
    W = torch.from_numpy(synth.make_blocks(fmt, N, K, seed=1)).cuda()
    X = torch.from_numpy(synth.make_activations(M, K, seed=2)).cuda()
    assert torch.equal(ops.gemm_static(fmt, W, X, N), ops.gemm(fmt, W, X, N))


@pytest.mark.gpu
def test_static_refuses_oversize_on_device():
    import torch
    from brotensor_b200 import ops
    fmt, N, K, M = synth.Q4_K, 128, 8192, 1040
    W = torch.from_numpy(synth.make_blocks(fmt, N, K, seed=1)).cuda()
    X = torch.zeros((M, K), device="cuda")
    with pytest.raises(_capi.B200QError) as e:
        ops.gemm_static(fmt, W, X, N)
    assert e.value.status == _capi.ERR_WORKSPACE

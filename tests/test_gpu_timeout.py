"""A bounded device-side wait that runs out: the sharded GEMV's wait for a peer rank that never
arrives. Nothing faults or hangs: the kernel gives up after the limit, records a status word and
returns; the host reads B200Q_ERR_TIMEOUT once, and the device goes on working."""
import ctypes as C

import numpy as np
import pytest

from brotensor_b200 import synth


@pytest.mark.gpu
def test_peer_wait_runs_out_and_the_device_stays_usable(cpu_oracle):
    import torch
    import oracle
    from brotensor_b200 import _capi as capi, ops
    L = capi.lib()
    fmt, rows, K = synth.Q4_K, 512, 1024
    world, total = 2, 2 * rows
    Wh = synth.make_blocks(fmt, rows, K, seed=31)
    xh = synth.make_activations(1, K, seed=31)
    W = torch.from_numpy(Wh).cuda()
    x = torch.from_numpy(xh).cuda()
    # rank 0 of 2 on one GPU: rank 1's exchange memory is a second local buffer that nobody ever writes
    # rows into, so rank 0's wait for rank 1's rows cannot complete
    # (two result vectors of floats + two vectors of 8-byte transfer words = 6 floats per row)
    outs = [torch.zeros(6 * total, dtype=torch.float32, device="cuda") for _ in range(world)]
    state = torch.zeros(4, dtype=torch.int32, device="cuda")
    po = (C.c_void_p * world)(*[t.data_ptr() for t in outs])
    assert ops.device_status() == 0
    ops.set_option("wait_limit_us", 2000)  # two milliseconds instead of a second
    try:
        stream = torch.cuda.current_stream().cuda_stream
        rc = L.b200q_gemv_shard(fmt, W.data_ptr(), x.data_ptr(), capi.F32, None, rows, K, 0, total, 0, world, po,
                                state.data_ptr(), stream)
        assert rc == capi.OK, L.b200q_last_error()
        torch.cuda.synchronize()  # the kernel returned by itself
        v = C.c_int(0)
        rc = L.b200q_device_status(C.byref(v))
        assert rc == capi.ERR_TIMEOUT and v.value == 105, (rc, v.value)
        assert b"wait" in L.b200q_last_error()
        rc = L.b200q_device_status(C.byref(v))  # reading the status resets it
        assert rc == capi.OK and v.value == 0
        # this rank's own rows did arrive in its result vector (call 1 -> vector 1), and at the "peer" as
        # transfer words (value, call number 1) behind its two result vectors
        want = cpu_oracle.matmul(fmt, Wh, xh, threads=4).reshape(-1)
        got = outs[0].cpu().numpy()[total:total + rows]
        assert oracle.rel_l2(got, want) < 2e-3
        words = outs[1].cpu().numpy()[2 * total:].view(np.uint32).reshape(2, total, 2)[1, :rows]
        assert np.array_equal(words[:, 0].view(np.float32), got) and np.all(words[:, 1] == 1)
        assert int(state.cpu()[1]) == 1
    finally:
        ops.set_option("wait_limit_us", 0)
    # the device is as usable as before: a plain GEMV right after the timeout
    y = ops.gemv(fmt, W, x, rows).cpu().numpy().reshape(-1)
    assert oracle.rel_l2(y, want) < 2e-3
    assert ops.device_status() == 0

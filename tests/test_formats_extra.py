"""Q4_0 and Q5_K (GGUF formats that brotensor's loader carries without an op) and the quantized
embedding-row gather.

The reference has no decoder for the two formats, so there are no reference vectors to pin them
to: the C oracle restates ggml's block definitions, and the numpy functions below restate them a
second time, written separately; the CPU test checks that the two agree bit for bit, the GPU tests
check the kernels against the oracle (decode bitwise, GEMV rel-L2 <= 2e-3)."""
import numpy as np
import pytest

import oracle
from brotensor_b200 import synth


def np_dequant_q4_0(W, rows, K):
    b = W.reshape(rows * (K // 32), 18)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float32)            # (nb, 1)
    qs = b[:, 2:18].astype(np.int32)
    lo, hi = (qs & 15) - 8, (qs >> 4) - 8
    return (d * np.concatenate([lo, hi], axis=1).astype(np.float32)).reshape(rows, K)


def np_dequant_q5k(W, rows, K):
    b = W.reshape(rows * (K // 256), 176)
    nb = b.shape[0]
    d = b[:, 0:2].copy().view(np.float16).astype(np.float32)
    dmin = b[:, 2:4].copy().view(np.float16).astype(np.float32)
    s = b[:, 4:16].astype(np.int32)
    sc = np.empty((nb, 8), np.int32)
    m = np.empty((nb, 8), np.int32)
    sc[:, :4], m[:, :4] = s[:, 0:4] & 63, s[:, 4:8] & 63
    sc[:, 4:] = (s[:, 8:12] & 15) | ((s[:, 0:4] >> 6) << 4)
    m[:, 4:] = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
    qh = b[:, 16:48].astype(np.int32)
    ql = b[:, 48:176].astype(np.int32).reshape(nb, 4, 32)
    out = np.empty((nb, 8, 32), np.float32)
    for sub in range(8):
        j = sub // 2
        nib = (ql[:, j, :] >> 4) if (sub & 1) else (ql[:, j, :] & 15)
        q = nib + 16 * ((qh >> sub) & 1)
        # two exact products and one rounding, as in the C oracle
        out[:, sub, :] = (d * sc[:, sub:sub + 1].astype(np.float32)) * q.astype(np.float32) - dmin * m[:, sub:sub + 1].astype(np.float32)
    return out.reshape(rows, K)


CASES = [(synth.Q4_0, np_dequant_q4_0, 37, 512), (synth.Q5_K, np_dequant_q5k, 19, 1024)]


@pytest.mark.parametrize("fmt,np_deq,rows,K", CASES)
def test_oracle_agrees_with_the_numpy_restatement(fmt, np_deq, rows, K, cpu_oracle):
    W = synth.make_blocks(fmt, rows, K, seed=fmt)
    a = cpu_oracle.dequant_f32(fmt, W, rows, K)
    b = np_deq(W, rows, K)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_q5k_known_block(cpu_oracle):
    """One hand-built block: d = 1, dmin = 0.5, every scale 2 and min 4, quants chosen so that the
    expected values are easy to write down."""
    blk = np.zeros(176, np.uint8)
    blk[0:2] = np.array([1.0], np.float16).view(np.uint8)
    blk[2:4] = np.array([0.5], np.float16).view(np.uint8)
    sc = np.full(8, 2, np.uint8)
    m = np.full(8, 4, np.uint8)
    s = np.zeros(12, np.uint8)
    cpu_oracle.lib.oracle_q4k_pack_sc_m(s.ctypes.data_as(oracle._u8p), sc.ctypes.data_as(oracle._u8p), m.ctypes.data_as(oracle._u8p))
    blk[4:16] = s
    blk[48:176] = 0x21          # low nibble 1, high nibble 2
    blk[16:48] = 0b00000101     # fifth bit set for sub-blocks 0 and 2
    got = cpu_oracle.dequant_f32(synth.Q5_K, blk, 1, 256).reshape(8, 32)
    want = np.array([2 * (1 + 16) - 2, 2 * 2 - 2, 2 * (1 + 16) - 2, 2 * 2 - 2, 2 * 1 - 2, 2 * 2 - 2, 2 * 1 - 2, 2 * 2 - 2], np.float32)
    assert np.array_equal(got, np.repeat(want[:, None], 32, axis=1))


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,rows,K", [(synth.Q4_0, 300, 4096), (synth.Q5_K, 300, 4096), (synth.Q5_K, 70001, 256), (synth.Q4_0, 5, 32)])
def test_decode_is_bit_exact(fmt, rows, K, cpu_oracle):
    import torch
    from brotensor_b200 import ops
    if K % 8:
        pytest.skip("rows shorter than one decode unit")
    Wh = synth.make_blocks(fmt, rows, K, seed=rows)
    W = torch.from_numpy(Wh).cuda()
    f32 = ops.dequant(fmt, W, rows, K, torch.float32).cpu().numpy()
    assert np.array_equal(f32.view(np.uint32), cpu_oracle.dequant_f32(fmt, Wh, rows, K).view(np.uint32))
    f16 = ops.dequant(fmt, W, rows, K, torch.float16).cpu().numpy()
    assert np.array_equal(f16.view(np.uint16), cpu_oracle.dequant_16(fmt, Wh, rows, K, 1))
    bf = ops.dequant(fmt, W, rows, K, torch.bfloat16).view(torch.int16).cpu().numpy()
    assert np.array_equal(bf.view(np.uint16), cpu_oracle.dequant_16(fmt, Wh, rows, K, 4))
    assert ops.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", [synth.Q4_0, synth.Q5_K])
@pytest.mark.parametrize("M", [1, 3, 8, 20])
def test_linear_matches_the_oracle(fmt, M, cpu_oracle):
    import torch
    from brotensor_b200 import ops
    N, K = 777, 2048
    Wh = synth.make_blocks(fmt, N, K, seed=M)
    Xh = synth.make_activations(M, K, seed=M)
    bias = synth.make_activations(1, N, seed=9).reshape(-1)
    W, X, b = torch.from_numpy(Wh).cuda(), torch.from_numpy(Xh).cuda(), torch.from_numpy(bias).cuda()
    want = cpu_oracle.matmul(fmt, Wh, Xh, bias=bias, threads=4)
    got = ops.linear(fmt, W, X, N, bias=b).cpu().numpy()   # M <= 8: decode GEMV; above: passes of the GEMV
    assert oracle.rel_l2(got, want) < 2e-3
    # FP16 activations and results (the reference's contract for its own formats)
    got16 = ops.linear(fmt, W, X.half(), N, bias=b.half()).float().cpu().numpy()
    assert oracle.rel_l2(got16, want) < 5e-3
    assert ops.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", [synth.Q4_K, synth.Q6_K, synth.Q8_0, synth.Q4_0, synth.Q5_K])
def test_embedding_gather_is_the_dequant_of_the_rows(fmt, cpu_oracle):
    import torch
    from brotensor_b200 import ops
    rows, K = 1000, 2048
    Wh = synth.make_blocks(fmt, rows, K, seed=77)
    W = torch.from_numpy(Wh).cuda()
    idx_h = np.array([0, 999, 5, 5, 123, -1, 1000, 42, 2 ** 31 - 1], np.int32)   # repeats, both ends, three invalid
    idx = torch.from_numpy(idx_h).cuda()
    full16 = cpu_oracle.dequant_16(fmt, Wh, rows, K, 1)
    full32 = cpu_oracle.dequant_f32(fmt, Wh, rows, K)
    valid = (idx_h >= 0) & (idx_h < rows)
    for dt, full in ((torch.float16, full16), (torch.float32, full32.view(np.uint32))):
        got = ops.embedding_gather(fmt, W, idx, rows, K, dt).cpu().numpy()
        got = got.view(np.uint16) if dt == torch.float16 else got.view(np.uint32)
        for i, r in enumerate(idx_h):
            if valid[i]:
                assert np.array_equal(got[i], full[r]), (i, r)
            else:
                assert not got[i].any()                      # outside the table: zeros, nothing read
    empty = ops.embedding_gather(fmt, W, idx[:0].contiguous(), rows, K)
    assert empty.shape == (0, K)
    assert ops.device_status() == 0


@pytest.mark.gpu
def test_fused_forms_refuse_the_extra_formats():
    import torch
    from brotensor_b200 import _capi as capi, ops
    N, K = 64, 256
    W = torch.from_numpy(synth.make_blocks(synth.Q5_K, N, K, seed=1)).cuda()
    x = torch.zeros(K, device="cuda")
    with pytest.raises(capi.B200QError) as e:
        ops.gemv_swiglu(synth.Q5_K, W, W, x, N)
    assert e.value.status == capi.ERR_UNSUPPORTED

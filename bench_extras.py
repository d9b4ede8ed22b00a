"""Secondary measurements of bench.py: the benchmark configurations other than the
headline decode layer set. Every number is parity-gated against the CPU oracle by the
caller's tests; here only timing happens (CUDA events around CUDA-graph replays that
rotate over weight replicas larger than the L2).

  config0   Q4_K 4096x4096, M=1 GEMV                      GB/s of packed weight bytes
  config2   Q8_0 14336x4096, M in {1,2,4,8}               GB/s (weights counted once)
  config3   Q4_K 14336x4096 prefill GEMM, M=512 tokens    TFLOP/s vs the measured bf16 peak
  lm_head   Q6_K 128256x4096 rows split over the ranks, per-shard GEMV + NCCL all-gather
            of the fp32 logits; tok/s = 1 / time of the slowest rank
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

from brotensor_b200 import ops, shard, synth


def _time_graph(fn, n_launch, stream, reps=10):
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        for i in range(n_launch):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ts = []
    for _ in range(reps):
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) / n_launch)
    return float(np.median(ts)), float(np.min(ts))  # ms per launch


def _replicas(fmt, N, K, seed, budget_bytes=1.2e9, cap=32, want_host=False):
    nbytes = synth.packed_bytes(fmt, N, K)
    R = int(max(2, min(cap, budget_bytes // nbytes)))
    host = synth.make_blocks(fmt, N, K, seed=seed)
    base = torch.from_numpy(host).cuda()
    reps = [base] + [torch.roll(base, 1028160 * (i + 1)).contiguous() for i in range(R - 1)]
    return (reps, nbytes, host) if want_host else (reps, nbytes)


def gemv_case(fmt, N, K, M, stream, peak_gbs, n_launch=48):
    Ws, nbytes = _replicas(fmt, N, K, seed=N + K)
    X = torch.from_numpy(synth.make_activations(M, K, seed=M)).cuda()
    Y = torch.empty((M, N), dtype=torch.float32, device="cuda")
    for i in range(3):
        ops.gemv(fmt, Ws[i % len(Ws)], X, N, out=Y)
    med, mn = _time_graph(lambda i: ops.gemv(fmt, Ws[i % len(Ws)], X, N, out=Y), n_launch, stream)
    gbs = nbytes / (med * 1e-3) / 1e9
    return {"fmt": synth.FMT_NAME[fmt], "N": N, "K": K, "M": M, "us": med * 1e3, "us_min": mn * 1e3, "GBps": gbs,
            "frac_of_hbm_peak": gbs / peak_gbs, "replicas": len(Ws)}


def gemm_case(fmt, N, K, M, x_dtype, stream, peaks, n_launch=8, regrouped=False):
    W = torch.from_numpy(synth.make_blocks(fmt, N, K, seed=3)).cuda()
    if regrouped:  # the device-side regrouped layout of the same blocks (b200q_repack)
        W = ops.repack(fmt, W, N, K)
        fmt = ops.repacked_fmt(fmt, K)
    X = torch.from_numpy(synth.make_activations(M, K, seed=3)).cuda().to(x_dtype)
    Y = torch.empty((M, N), dtype=torch.float32, device="cuda")
    from brotensor_b200 import _capi
    need = _capi.lib().b200q_gemm_workspace_bytes(fmt, ops._DT[x_dtype], M, N, K)
    ws = torch.empty(max(need, 256), dtype=torch.uint8, device="cuda")
    for _ in range(3):
        ops.gemm(fmt, W, X, N, out=Y, ws=ws)
    ops.tc_calls_consume(fmt)
    med, mn = _time_graph(lambda i: ops.gemm(fmt, W, X, N, out=Y, ws=ws), n_launch, stream)
    tc = ops.tc_calls_consume(fmt)
    flops = 2.0 * M * N * K
    tf = flops / (med * 1e-3) / 1e12
    return {"fmt": synth.FMT_NAME[fmt], "N": N, "K": K, "M": M, "x_dtype": str(x_dtype).replace("torch.", ""),
            "us": med * 1e3, "us_min": mn * 1e3, "TFLOPs": tf, "frac_of_bf16_burst_peak": tf / peaks["bf16_tflops"],
            "frac_of_bf16_sustained_peak": tf / peaks["bf16_tflops_sustained"] if peaks.get("bf16_tflops_sustained") else None,
            "tensor_core_launches": tc, "includes": "activation pre-pass (fp16 operand image) + tcgen05 GEMM"}


def lm_head_case(rank, world, stream, peak_gbs, n_launch=16):
    """Config 4: vocab rows split evenly over the ranks; every rank streams its own shard
    and the fp32 logits are all-gathered. Strong scaling: the total work is fixed."""
    fmt, N, K = synth.Q6_K, 128256, 4096
    b, e = shard.row_range(N, world, rank, align=16)
    rows = e - b
    assert rows * world == N, "the LM-head benchmark wants equal shards"
    # each rank generates only its shard (seeded per shard, so the content is independent of world size
    # only in distribution; parity of the sharded path is covered by the tests)
    Ws, nbytes, W_host = _replicas(fmt, rows, K, seed=4000 + rank, budget_bytes=1.0e9, cap=6, want_host=True)
    x_host = synth.make_activations(1, K, seed=4)
    x = torch.from_numpy(x_host).cuda()
    local = torch.empty((1, rows), dtype=torch.float32, device="cuda")
    full = torch.empty((world, rows), dtype=torch.float32, device="cuda")
    # parity gate before anything is timed: this rank's shard against the CPU oracle on its own rows
    import os
    import oracle
    ops.gemv(fmt, Ws[0], x, rows, out=local)
    torch.cuda.synchronize()
    err = oracle.rel_l2(local.cpu().numpy(), oracle.cpu().matmul(fmt, W_host, x_host, threads=max(1, (os.cpu_count() or 1) // max(world, 1))))
    del W_host
    e_t = torch.tensor([err], device="cuda")
    if world > 1:
        dist.all_reduce(e_t, op=dist.ReduceOp.MAX)
    err = float(e_t.item())
    assert err < 2e-3, f"LM-head shard parity failed: rel-L2 {err}"

    def step(i):
        ops.gemv(fmt, Ws[i % len(Ws)], x, rows, out=local)
        if world > 1:  # shard.all_gather_rows's equal-shard case, with the output preallocated
            dist.all_gather_into_tensor(full.view(-1), local.view(-1))

    for i in range(3):
        step(i)
    torch.cuda.synchronize()
    out = {"fmt": "q6k", "N": N, "K": K, "ranks": world, "rows_per_rank": rows, "oracle_rel_l2": err}
    # the gather cannot be captured on every NCCL configuration; fall back to stream launches
    try:
        med, mn = _time_graph(step, n_launch, stream)
        out["timed_as"] = "cuda graph"
    except Exception:  # noqa: BLE001
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ts = []
        for _ in range(5):
            e0.record()
            for i in range(n_launch):
                step(i)
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / n_launch)
        med, mn = float(np.median(ts)), float(np.min(ts))
        out["timed_as"] = "stream launches"
    t = torch.tensor([med], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    med = float(t.item())
    # GEMV alone, for the split between streaming and exchange
    g_med, _ = _time_graph(lambda i: ops.gemv(fmt, Ws[i % len(Ws)], x, rows, out=local), n_launch, stream)
    step(0)  # the gathered form on replica 0: the fused form must reproduce it
    torch.cuda.synchronize()
    out["fused"] = _fused_head(fmt, rows, K, b, N, rank, world, Ws, x, stream, n_launch, full if world > 1 else local)
    out.update({"us_per_token": med * 1e3, "tok_per_s": 1.0 / (med * 1e-3), "gemv_only_us": g_med * 1e3,
                "shard_GBps": nbytes / (g_med * 1e-3) / 1e9, "shard_frac_of_hbm_peak": nbytes / (g_med * 1e-3) / 1e9 / peak_gbs,
                "all_gather_bytes": 4 * N, "collective": "nccl all_gather_into_tensor" if world > 1 else "none"})
    return out


def _fused_head(fmt, rows, K, row0, N, rank, world, Ws, x, stream, n_launch, ref_full):
    """The one-kernel form: the shard GEMV stores its rows into every rank's result vector over
    NVLink and signals arrival itself (brotensor_b200::ShardedHead); no collective call."""
    from brotensor_b200 import hostapi
    try:
        hostapi.init()
        dev = torch.cuda.current_device()
        # the head's weights are Tensors of the host layer; they alias the replicas already on the device
        weights = [hostapi.Weight.view(fmt, w.data_ptr(), rows, K, dev) for w in Ws]

        def exchange(h):
            outl = [None] * world
            dist.all_gather_object(outl, h)
            return outl

        head = hostapi.ShardedHead(weights[0], row0, N, rank, world, exchange if world > 1 else None)
        hostapi.set_stream(torch.cuda.current_stream().cuda_stream, dev)
        # parity with the gathered form first: same kernel arithmetic, so bitwise
        head.run(x.data_ptr(), K, 0, weights[0])
        same = bool(np.array_equal(head.logits(), ref_full.reshape(-1).cpu().numpy()))
        if world > 1:
            dist.barrier()

        def step(i):
            head.run(x.data_ptr(), K, 0, weights[i % len(weights)])

        hostapi.set_stream(stream.cuda_stream, dev)
        med, mn = _time_graph(step, n_launch, stream)
        hostapi.set_stream(torch.cuda.current_stream().cuda_stream, dev)
        t = torch.tensor([med], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        med = float(t.item())
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        # the greedy-sampling form: one (value, row) candidate per rank crosses the links instead of the logits
        head.run_topk(x.data_ptr(), K, 1, 0, weights[0])
        tv, tr = head.top(1)
        ref = ref_full.reshape(-1).cpu().numpy()
        best = int(np.lexsort((np.arange(ref.size), -ref))[0])
        greedy_ok = bool(int(tr[0]) == best and tv[0] == ref[best])
        if world > 1:
            dist.barrier()

        def step_top(i):
            head.run_topk(x.data_ptr(), K, 1, 0, weights[i % len(weights)])

        hostapi.set_stream(stream.cuda_stream, dev)
        gmed, _ = _time_graph(step_top, n_launch, stream)
        hostapi.set_stream(torch.cuda.current_stream().cuda_stream, dev)
        t = torch.tensor([gmed], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        gmed = float(t.item())
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        status = ops.device_status()
        head.close()
        return {"us_per_token": med * 1e3, "tok_per_s": 1.0 / (med * 1e-3), "matches_gathered_bitwise": same,
                "greedy": {"us_per_token": gmed * 1e3, "tok_per_s": 1.0 / (gmed * 1e-3), "matches_argmax_of_gathered": greedy_ok,
                           "exchange": "one (value, row) candidate per rank; argmax of the whole vocabulary on every rank"},
                "device_status": status, "exchange": "peer stores + one release-add per CTA and peer inside the GEMV kernel (CUDA IPC memory)"}
    except Exception as ex:  # noqa: BLE001
        return {"error": repr(ex)}


def dequant_case(fmt, N, K, stream, peak_gbs, R=6, n_launch=12):
    """Decode to FP16 (the reference's dequant_*_to_fp16): bytes = packed read + FP16 written."""
    from brotensor_b200 import _capi
    W = torch.from_numpy(synth.make_blocks(fmt, N, K, seed=2)).cuda()
    outs = [torch.empty((N, K), dtype=torch.float16, device="cuda") for _ in range(R)]  # R x 32 MiB > L2

    def run(i):
        _capi.check(_capi.lib().b200q_dequant(fmt, W.data_ptr(), outs[i % R].data_ptr(), 1, N, K, torch.cuda.current_stream().cuda_stream))

    for i in range(3):
        run(i)
    med, mn = _time_graph(run, n_launch, stream)
    nbytes = synth.packed_bytes(fmt, N, K) + 2 * N * K
    gbs = nbytes / (med * 1e-3) / 1e9
    return {"fmt": synth.FMT_NAME[fmt], "N": N, "K": K, "us": med * 1e3, "GBps_read_plus_written": gbs, "frac_of_hbm_peak": gbs / peak_gbs}


def grouped_layer_set(stream, peak_gbs, R=8, n_steps=24):
    """The decode layer set with the GEMVs that share an activation vector fused into one launch
    each (b200q_gemv_multi): [q, k, v], o, [gate, up], down - four launches instead of seven."""
    specs = synth.LLAMA3_8B_LAYER_SET
    host = [synth.make_blocks(fmt, N, K, seed=100 + i) for i, (_, fmt, N, K) in enumerate(specs)]
    reps = []
    for r in range(R):
        reps.append([(torch.roll(torch.from_numpy(W).cuda(), r * 1028160).contiguous() if r else torch.from_numpy(W).cuda()) for W in host])
    idx = {name: i for i, (name, _, _, _) in enumerate(specs)}
    x4 = torch.from_numpy(synth.make_activations(1, 4096, seed=1)).cuda().view(-1)
    x14 = torch.from_numpy(synth.make_activations(1, 14336, seed=2)).cuda().view(-1)
    outs = [torch.empty((1, N), dtype=torch.float32, device="cuda") for _, _, N, _ in specs]
    groups = [["q_proj", "k_proj", "v_proj"], ["o_proj"], ["gate_proj", "up_proj"], ["down_proj"]]

    def step(r):
        Wr = reps[r % R]
        for g in groups:
            ii = [idx[n] for n in g]
            fmt, K = specs[ii[0]][1], specs[ii[0]][3]
            x = x14 if K == 14336 else x4
            if len(ii) == 1:
                ops.gemv(fmt, Wr[ii[0]], x, specs[ii[0]][2], out=outs[ii[0]])
            else:
                ops.gemv_multi(fmt, [Wr[i] for i in ii], x, [specs[i][2] for i in ii], outs=[outs[i] for i in ii])

    for i in range(3):
        step(i)
    med, mn = _time_graph(step, n_steps, stream)
    nbytes = sum(synth.packed_bytes(f, n, k) for _, f, n, k in specs)
    gbs = nbytes / (med * 1e-3) / 1e9
    # the gate / up pair alone: two launches, one grouped launch, one launch with the SwiGLU gate folded in
    ig, iu = idx["gate_proj"], idx["up_proj"]
    fmt_g, n_g = specs[ig][1], specs[ig][2]
    act = torch.empty((1, n_g), dtype=torch.float32, device="cuda")

    def two(r):
        ops.gemv(fmt_g, reps[r % R][ig], x4, n_g, out=outs[ig])
        ops.gemv(fmt_g, reps[r % R][iu], x4, n_g, out=outs[iu])

    def one(r):
        ops.gemv_multi(fmt_g, [reps[r % R][ig], reps[r % R][iu]], x4, [n_g, n_g], outs=[outs[ig], outs[iu]])

    def gated(r):
        ops.gemv_swiglu(fmt_g, reps[r % R][ig], reps[r % R][iu], x4, n_g, out=act)

    pair = {}
    for name, f in (("two_launches_us", two), ("grouped_us", one), ("swiglu_fused_us", gated)):
        for i in range(3):
            f(i)
        pair[name] = _time_graph(f, n_steps, stream)[0] * 1e3
    # q / k / v grouped, without and with the RMSNorm of their input folded into the launch
    iq = [idx["q_proj"], idx["k_proj"], idx["v_proj"]]
    gamma = torch.ones(4096, dtype=torch.float32, device="cuda")

    def qkv(r):
        ops.gemv_multi(specs[iq[0]][1], [reps[r % R][i] for i in iq], x4, [specs[i][2] for i in iq], outs=[outs[i] for i in iq])

    def qkv_norm(r):
        ops.gemv_multi_rmsnorm(specs[iq[0]][1], [reps[r % R][i] for i in iq], x4, gamma, 1e-5, [specs[i][2] for i in iq], outs=[outs[i] for i in iq])

    for name, f in (("qkv_grouped_us", qkv), ("qkv_grouped_rmsnorm_folded_us", qkv_norm)):
        for i in range(3):
            f(i)
        pair[name] = _time_graph(f, n_steps, stream)[0] * 1e3
    pair["packed_bytes"] = 2 * synth.packed_bytes(fmt_g, n_g, 4096)
    pair["swiglu_fused_GBps"] = pair["packed_bytes"] / (pair["swiglu_fused_us"] * 1e-6) / 1e9
    return {"launches_per_step": 4, "us_per_step": med * 1e3, "GBps": gbs, "frac_of_hbm_peak": gbs / peak_gbs,
            "fused_pieces": pair,
            "note": "same seven matrix-vector products as the headline; the headline keeps one launch per op "
                    "because that is the reference's op interface"}


def repack_case(stream, peak_gbs, N=4096, K=14336, R=12):
    """Q6_K down_proj in the GGUF layout against the device-side regrouped one (b200q_repack):
    the repack pass itself, the decode GEMV and the decode to FP16 on both layouts."""
    from brotensor_b200 import _capi
    fmt, pf = synth.Q6_K, synth.Q6_K_R8
    base = torch.from_numpy(synth.make_blocks(fmt, N, K, seed=9)).cuda()
    raw = [base] + [torch.roll(base, 1680 * 97 * (i + 1)).contiguous() for i in range(R - 1)]
    packed = [ops.repack(fmt, w, N, K) for w in raw]
    nbytes = synth.packed_bytes(fmt, N, K)
    assert torch.equal(ops.unpack(fmt, packed[1], N, K), raw[1])
    x = torch.from_numpy(synth.make_activations(1, K, seed=2)).cuda()
    y = torch.empty((1, N), dtype=torch.float32, device="cuda")
    res = {"fmt": "q6k", "N": N, "K": K, "round_trip_bit_identical": True}
    for name, f, ws in (("gguf_layout", fmt, raw), ("regrouped", pf, packed)):
        def gv(i):
            ops.gemv(f, ws[i % R], x, N, out=y)
        for i in range(3):
            gv(i)
        med, _ = _time_graph(gv, 48, stream)
        res["gemv_us_" + name] = med * 1e3
    assert torch.equal(ops.gemv(pf, packed[0], x, N), ops.gemv(fmt, raw[0], x, N))
    scratch = torch.empty_like(base)

    def rp(i):
        _capi.check(_capi.lib().b200q_repack(fmt, raw[i % R].data_ptr(), scratch.data_ptr(), N, K, torch.cuda.current_stream().cuda_stream))
    for i in range(3):
        rp(i)
    med, _ = _time_graph(rp, 12, stream)
    res["repack_us"] = med * 1e3
    res["repack_GBps_read_plus_written"] = 2 * nbytes / (med * 1e-3) / 1e9
    res["note"] = ("opt-in at load (brotensor_b200::repack_weights, gguf::upload_rows_repacked): a regrouped weight has no "
                   "raw host image to read back, so the loader keeps the GGUF layout unless asked")
    return res


def reference_cuda(peaks, stream, root):
    """brotensor's OWN CUDA quant kernels (src/cuda/q4k.cu, q6k.cu, q8_0.cu and the WMMA prefill files)
    compiled unmodified for sm_100a into oracle/_ref/libref_cuda.so and called through brotensor's public
    ops (FP16 activations and outputs, the only dtype that API has) on the same box: the decode layer
    set, config 2 and the prefill shape, timed like this repository's own arm (CUDA events around graph
    replays that rotate over weight replicas larger than the L2). Reference arm only."""
    import ctypes
    import os
    path = os.path.join(root, "oracle", "_ref", "libref_cuda.so")
    if not os.path.exists(path):
        return {"unavailable": "oracle/_ref/libref_cuda.so not built (make -C oracle gpu)"}
    lib = ctypes.CDLL(path)
    lib.refcuda_last_error.restype = ctypes.c_char_p
    lib.refcuda_linear.argtypes = [ctypes.c_int] + [ctypes.c_void_p] * 3 + [ctypes.c_int] * 3
    lib.refcuda_set_stream.argtypes = [ctypes.c_void_p]
    if not lib.refcuda_init():
        return {"unavailable": "brotensor's CUDA backend did not register: " + lib.refcuda_last_error().decode()}
    tag = {synth.Q4_K: 22, synth.Q6_K: 24, synth.Q8_0: 14}  # brotensor::Dtype (include/brotensor/tensor.h:17-33)

    def linear(fmt, W, X, Y, B, N, K):
        if lib.refcuda_linear(tag[fmt], W.data_ptr(), X.data_ptr(), Y.data_ptr(), B, N, K):
            raise RuntimeError("brotensor: " + lib.refcuda_last_error().decode())

    def timed(fn, n_launch):
        lib.refcuda_set_stream(torch.cuda.current_stream().cuda_stream)
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            lib.refcuda_set_stream(s.cuda_stream)
            try:
                med, mn = _time_graph(fn, n_launch, s)
                how = "graph"
            finally:
                lib.refcuda_set_stream(torch.cuda.current_stream().cuda_stream)
        return med, mn, how

    def case(fmt, N, K, M, n_launch=24):
        Ws, nbytes = _replicas(fmt, N, K, seed=N + K)
        X = torch.from_numpy(synth.make_activations(M, K, seed=M)).cuda().half()
        Y = torch.empty((M, N), dtype=torch.float16, device="cuda")
        med, mn, how = timed(lambda i: linear(fmt, Ws[i % len(Ws)], X, Y, M, N, K), n_launch)
        r = {"fmt": synth.FMT_NAME[fmt], "N": N, "K": K, "M": M, "us": med * 1e3, "us_min": mn * 1e3, "timing": how}
        if M <= 8:
            r["GBps"] = nbytes / (med * 1e-3) / 1e9
            r["frac_of_hbm_peak"] = r["GBps"] / peaks["hbm_gbs"]
        else:
            r["TFLOPs"] = 2.0 * M * N * K / (med * 1e-3) / 1e12
            r["frac_of_bf16_burst_peak"] = r["TFLOPs"] / peaks["bf16_tflops"]
        # the numbers of a wrong kernel are worth nothing: compare against this repository's checked path
        ref = torch.empty((M, N), dtype=torch.float32, device="cuda")
        (ops.gemv if M <= 8 else ops.gemm)(fmt, Ws[0], X.float(), N, out=ref)
        linear(fmt, Ws[0], X, Y, M, N, K)
        torch.cuda.synchronize()
        r["rel_l2_vs_this_repo"] = float((Y.float() - ref).norm() / ref.norm())
        return r

    out = {"what": "brotensor src/cuda quant kernels, unmodified, nvcc -gencode arch=compute_100a,code=sm_100a, "
                   "through brotensor's public ops (FP16 x and y)"}
    per = [case(fmt, N, K, 1) | {"name": name} for name, fmt, N, K in synth.LLAMA3_8B_LAYER_SET]
    out["layer_set_per_kernel"] = per
    total_us = sum(c["us"] for c in per)
    layer_bytes = sum(synth.packed_bytes(f, n, k) for _, f, n, k in synth.LLAMA3_8B_LAYER_SET)
    out["layer_set"] = {"us": total_us, "GBps": layer_bytes / (total_us * 1e-6) / 1e9,
                        "note": "sum of the seven per-kernel times (each kernel timed back to back with itself)"}
    out["config2_q8_0_14336x4096"] = [case(synth.Q8_0, 14336, 4096, M) for M in (1, 2, 4, 8)]
    out["config3_prefill_512"] = [case(f, 14336, 4096, 512, n_launch=6) for f in (synth.Q4_K, synth.Q6_K, synth.Q8_0)]
    return out


def upload_case(N=57344, K=4096):
    """Weight upload from a GGUF file (page cache warm): the host layer's staged upload (two pinned 8 MiB
    buffers, memcpy of the next piece overlapping the DMA of the previous one; gguf::upload_rows) against one
    blocking cudaMemcpy from the pageable mapping, which is what brotensor's upload_raw does
    (src/gguf.cpp:473-500 through Tensor::from_raw_bytes_on)."""
    import ctypes as C
    import os
    import struct
    import tempfile
    import time
    from brotensor_b200 import hostapi
    hostapi.init()
    L = hostapi.lib()
    fmt = synth.Q4_K
    payload = synth.make_blocks(fmt, N, K, seed=11).tobytes()
    align, name, key = 32, b"blk.0.ffn_gate.weight", b"general.alignment"
    head = struct.pack("<IIQQ", 0x46554747, 3, 1, 1) + struct.pack("<Q", len(key)) + key + struct.pack("<II", 4, align)
    head += struct.pack("<Q", len(name)) + name + struct.pack("<I", 2) + struct.pack("<QQ", K, N) + struct.pack("<IQ", 12, 0)  # 12 = GGML_TYPE_Q4_K
    head += b"\0" * ((align - len(head) % align) % align)
    fd, path = tempfile.mkstemp(suffix=".gguf")
    try:
        with os.fdopen(fd, "wb") as f:
            f.write(head + payload)
        L.b200h_gguf_open.restype = C.c_void_p
        L.b200h_gguf_open.argtypes = [C.c_char_p]
        L.b200h_gguf_close.argtypes = [C.c_void_p]
        L.b200h_gguf_upload_rows.restype = C.c_void_p
        L.b200h_gguf_upload_rows.argtypes = [C.c_void_p] + [C.c_int] * 6
        L.b200h_tensor_free.argtypes = [C.c_void_p]
        h = L.b200h_gguf_open(path.encode())
        assert h, L.b200h_last_error()
        dev = torch.cuda.current_device()
        staged = []
        for _ in range(4):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            t = L.b200h_gguf_upload_rows(h, 0, N, K, 0, N, dev)  # returns when the bytes are on the device
            staged.append(time.perf_counter() - t0)
            assert t, L.b200h_last_error()
            L.b200h_tensor_free(t)
        L.b200h_gguf_close(h)
        mm = np.memmap(path, dtype=np.uint8, mode="c", offset=len(head), shape=(len(payload),))  # copy-on-write: pageable, never written
        dst = torch.empty(len(payload), dtype=torch.uint8, device="cuda")
        blocking = []
        for _ in range(4):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            dst.copy_(torch.from_numpy(mm))  # pageable source: one blocking copy
            torch.cuda.synchronize()
            blocking.append(time.perf_counter() - t0)
        same = bool(torch.equal(dst[:4096].cpu(), torch.frombuffer(bytearray(payload[:4096]), dtype=torch.uint8)))
        del mm
    finally:
        os.unlink(path)
    nb = len(payload)
    return {"fmt": "q4k", "N": N, "K": K, "bytes": nb, "staged_GBps": nb / min(staged[1:]) / 1e9, "staged_ms": min(staged[1:]) * 1e3,
            "blocking_pageable_GBps": nb / min(blocking[1:]) / 1e9, "blocking_ms": min(blocking[1:]) * 1e3, "bytes_checked": same,
            "note": "file in the page cache; best of three after one warm-up; host time from call to bytes resident"}


def run(rank, world, peaks, stream):
    out = {}
    if world == 1:
        out["config0_q4k_4096x4096_m1"] = gemv_case(synth.Q4_K, 4096, 4096, 1, stream, peaks["hbm_gbs"])
        out["layer_set_per_kernel"] = [gemv_case(fmt, N, K, 1, stream, peaks["hbm_gbs"]) | {"name": name}
                                       for name, fmt, N, K in synth.LLAMA3_8B_LAYER_SET if name not in ("v_proj", "up_proj", "o_proj")]
        out["config2_q8_0_14336x4096"] = [gemv_case(synth.Q8_0, 14336, 4096, M, stream, peaks["hbm_gbs"]) for M in (1, 2, 4, 8)]
        out["small_batch_q4k_14336x4096"] = [gemv_case(synth.Q4_K, 14336, 4096, M, stream, peaks["hbm_gbs"]) for M in (2, 4, 8)]
        out["config3_q4k_prefill_512"] = [gemm_case(synth.Q4_K, 14336, 4096, 512, dt, stream, peaks)
                                          for dt in (torch.float32, torch.bfloat16)]
        out["prefill_other_formats_512"] = [gemm_case(f, 14336, 4096, 512, torch.float32, stream, peaks) for f in (synth.Q6_K, synth.Q8_0)]
        out["prefill_q6k_regrouped_512"] = gemm_case(synth.Q6_K, 14336, 4096, 512, torch.float32, stream, peaks, regrouped=True)
        # the other matrices of the layer at 512 tokens: 32 and 8 row tiles, k range split over CTA pairs
        out["prefill_layer_set_512"] = [gemm_case(fmt, N, K, 512, torch.float32, stream, peaks, n_launch=6) | {"name": name}
                                        for name, fmt, N, K in synth.LLAMA3_8B_LAYER_SET if name in ("q_proj", "k_proj", "down_proj")]
        out["layer_set_grouped"] = grouped_layer_set(stream, peaks["hbm_gbs"])
        out["dequant_to_fp16_4096x4096"] = [dequant_case(f, 4096, 4096, stream, peaks["hbm_gbs"]) for f in (synth.Q4_K, synth.Q6_K, synth.Q8_0)]
        out["repack_q6k_down_proj"] = repack_case(stream, peaks["hbm_gbs"])
        try:
            out["upload_gguf_q4k_132MB"] = upload_case()
        except Exception as ex:  # noqa: BLE001 - a full /tmp must not cost the benchmark line
            out["upload_gguf_q4k_132MB"] = {"error": repr(ex)[:300]}
    out["lm_head"] = lm_head_case(rank, world, stream, peaks["hbm_gbs"])
    return out

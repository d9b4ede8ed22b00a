#!/usr/bin/env python
"""Benchmark of the GGUF fused quant-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (config.workload = "llama3_8b_decode_layer_set_m1"): one step is
one pass of the seven decode GEMVs of a Llama-3-8B-shaped layer at M=1 (six Q4_K
projections and the Q6_K down_proj) over seeded synthetic GGUF blocks; the metric
is packed quantized weight bytes streamed per second (GB/s), the numerator the
reference's own bench uses (tests/bench_quant_matmul.cpp:5-10,207-209).

  value     steps timed on the device with inputs resident in HBM; the K steps are
            captured in one CUDA graph that rotates over weight replicas whose
            combined size is several times the L2, so every launch streams cold weights.
  e2e       the same step through the C-ABI with HOST activation/result buffers:
            pinned host -> device copy of x, the seven GEMVs, device -> host read
            of the outputs, every step inside the timed region.
  roofline  the dominant kernel (Q4_K streaming GEMV on the gate/up shape) timed
            alone with CUDA events; algorithmic bytes / duration vs the measured HBM peak.
  extras    config 0 (single Q4_K 4096x4096 GEMV), config 2 (Q8_0, M=1..8), config 3
            (prefill GEMM) and config 4 (row-sharded LM head + all-gather) numbers.

With N > 1 (one process per GPU under torchrun) every rank runs its own replica of
the decode layer set on its own activations (weak scaling, no data-path collective)
and the ranks together run the row-sharded LM head, whose logits are all-gathered
over NCCL; that number is reported under extras.lm_head.

`--impl reference` times the reference's own CPU code for this path (its host
decode + sequential FP32 dot from its parity tests, built into oracle/_ref; the
oracle port when that library is absent) on all host cores, same metric and unit.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from brotensor_b200 import synth  # noqa: E402

WORKLOAD = "llama3_8b_decode_layer_set_m1"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel (the Q4_K decode
# GEMV on 14336x4096), from an ncu capture of `bench.py --case gemv:q4k:14336:4096:1`
DOMINANT_KERNEL_DRAM_TRAFFIC = 33069568
L2_BYTES = 126 * 1024 * 1024


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons while a region runs: NVML (read-only queries)
    from a thread every few milliseconds, nvidia-smi as the fallback."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.path = None
        self.thread = None
        self.stop_flag = threading.Event()
        self.sm, self.mx, self.reasons = [], [], set()

    def _nvml_loop(self, nv, h):
        while not self.stop_flag.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                bits = int(nv.nvmlDeviceGetCurrentClocksEventReasons(h))
                for bit, name in self.REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001
                break
            time.sleep(0.004)

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            # NVML enumerates physical devices; honour CUDA_VISIBLE_DEVICES when it lists ordinals
            vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            idx = self.index
            if vis and all(v.strip().isdigit() for v in vis.split(",")):
                idx = int(vis.split(",")[self.index])
            h = nv.nvmlDeviceGetHandleByIndex(idx)
            self.mx = [float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))]
            nv.nvmlDeviceGetCurrentClocksEventReasons(h)
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, h), daemon=True)
            self.thread.start()
            return
        except Exception:  # noqa: BLE001
            self.thread = None
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=f,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.thread is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            return {"sm_mhz": float(np.median(self.sm)) if self.sm else None, "sm_max_mhz": self.mx[0] if self.mx else None,
                    "samples": len(self.sm), "reasons": sorted(self.reasons), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1]))
                mx.append(float(c[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons), "source": "nvidia-smi"}


# --------------------------------------------------------------------------- reference arm (CPU)

def cpu_layer_set_pass(mat, threads, layers, acts):
    nbytes = 0
    for (name, fmt, N, K), W, x in zip(synth.LLAMA3_8B_LAYER_SET, layers, acts):
        mat(fmt, W, x, threads=threads)
        nbytes += W.size
    return nbytes


def run_cpu_arm(kind_wanted: str, steps: int, warmup: int, budget_s: float = 20.0):
    """Times the CPU implementation on a bounded sample: whole layer-set passes."""
    import oracle
    ref = oracle.ref() if kind_wanted == "reference" else None
    kind = "reference" if ref is not None else "port"
    mat = ref.matmul if ref is not None else oracle.cpu().matmul
    cores = os.cpu_count() or 1
    layers = [synth.make_blocks(fmt, N, K, seed=100 + i) for i, (_, fmt, N, K) in enumerate(synth.LLAMA3_8B_LAYER_SET)]
    acts = [synth.make_activations(1, K, seed=100 + i) for i, (_, _, _, K) in enumerate(synth.LLAMA3_8B_LAYER_SET)]
    t0 = time.perf_counter()
    nbytes = cpu_layer_set_pass(mat, cores, layers, acts)
    one = time.perf_counter() - t0
    # bounded: as many of the requested steps as fit in the time budget (at least one)
    w = max(0, min(warmup, int(2.0 / max(one, 1e-9))))
    k = max(1, min(steps, int(budget_s / max(one, 1e-9))))
    for _ in range(w):
        cpu_layer_set_pass(mat, cores, layers, acts)
    t0 = time.perf_counter()
    for _ in range(k):
        cpu_layer_set_pass(mat, cores, layers, acts)
    dt = time.perf_counter() - t0
    gbs = nbytes * k / dt / 1e9
    return {"value": gbs, "unit": "GB/s", "cores": cores, "kind": kind,
            "sample": f"{k} full passes of the 7-GEMV layer set ({nbytes} packed bytes each), {w} warm-up passes"}, k, w, dt / k * 1e3


# --------------------------------------------------------------------------- profiling drivers

_FMT = {"q4k": synth.Q4_K, "q6k": synth.Q6_K, "q8_0": synth.Q8_0}


def lm_head_summary(extras, world):
    """Strong-scaling result of the row-sharded LM head (config 4) lifted to the top level of the line:
    the headline `value` is the layer set run as independent replicas ("scaling": "weak"), which says
    nothing about sharding; this does."""
    lh = (extras or {}).get("lm_head") or {}
    if not lh:
        return None
    fused = lh.get("fused") or {}
    out = {"workload": "Q6_K 128256x4096 LM head, M=1, vocab rows split over the ranks (strong scaling)", "n_gpus": world,
           "variant": "one kernel: shard GEMV whose CTAs send their rows as self-validating words and receive the peers' slices" if "us_per_token" in fused else "shard GEMV + NCCL all-gather",
           "us_per_token": fused.get("us_per_token", lh.get("us_per_token")),
           "tok_per_s": fused.get("tok_per_s", lh.get("tok_per_s")),
           "nccl_all_gather_us_per_token": lh.get("us_per_token"), "shard_gemv_only_us": lh.get("gemv_only_us"),
           "oracle_rel_l2": lh.get("oracle_rel_l2"), "matches_gathered_bitwise": fused.get("matches_gathered_bitwise")}
    g = fused.get("greedy") or {}
    if g:
        out["greedy_us_per_token"] = g.get("us_per_token")
        out["greedy_matches_argmax_of_gathered"] = g.get("matches_argmax_of_gathered")
    # efficiency against one GPU needs the N = 1 line of the same box; the ideal is N x the one-GPU rate
    out["ideal_us_per_token_at_hbm_peak"] = synth.packed_bytes(synth.Q6_K, 128256, 4096) / max(world, 1) / (measured_peaks()["hbm_gbs"] * 1e3)
    return out


def run_case(spec: str, launches: int):
    """A few launches of one shape for a profiler: weights rotate over six replicas so that a captured
    launch streams from DRAM; a few hundred MB on the device at most."""
    import torch
    from brotensor_b200 import ops
    op, f, N, K, M = spec.split(":")
    fmt, N, K, M = _FMT[f], int(N), int(K), int(M)
    torch.cuda.set_device(0)
    base = torch.from_numpy(synth.make_blocks(fmt, N, K, seed=1)).cuda()
    Ws = [base] + [torch.roll(base, 1028160 * (i + 1)).contiguous() for i in range(5)]
    X = torch.from_numpy(synth.make_activations(M, K, seed=2)).cuda()
    Y = torch.empty((M, N), dtype=torch.float32, device="cuda")
    for i in range(launches):
        if op == "dequant":
            ops.dequant(fmt, Ws[i % len(Ws)], N, K, torch.float16)
        elif op == "gemm":
            ops.gemm(fmt, Ws[i % len(Ws)], X, N, out=Y)
        else:
            ops.gemv(fmt, Ws[i % len(Ws)], X, N, out=Y)
    torch.cuda.synchronize()
    print("device status", ops.device_status())


def run_phases(pdl=1, shapes="q4k:1024:4096,q4k:4096:4096,q4k:14336:4096,q6k:4096:14336"):
    """Where the time of a decode-GEMV launch goes, from %globaltimer stamps the trace build writes
    (per CTA: entry, barriers ready, predecessor complete, activations staged, first tile started,
    each pipeline's end, first and last weight copy issued). A CUDA graph chains 24 launches over
    cold weight replicas, as the benchmark does; times are relative to the end of the launch before."""
    import ctypes as C
    import torch
    from brotensor_b200 import _capi, ops
    L = _capi.lib()
    if not hasattr(L, "b200q_trace_set"):
        raise SystemExit("--phases needs the trace build: python -m brotensor_b200.build --trace, then "
                         "B200Q_LIB=brotensor_b200/lib/libb200q_trace.so python bench.py --phases")
    L.b200q_trace_set.argtypes = [C.c_void_p, C.c_int]
    L.b200q_trace_set.restype = None
    torch.cuda.set_device(0)
    ops.set_option("pdl", pdl)
    n_launch = 24
    rows = []
    for spec in shapes.split(","):
        fname, N, K = spec.split(":")
        fmt, N, K = {"q4k": synth.Q4_K, "q6k": synth.Q6_K, "q8_0": synth.Q8_0}[fname], int(N), int(K)
        nbytes = synth.packed_bytes(fmt, N, K)
        R = max(2, min(32, int(1.0e9 // nbytes)))
        base = torch.from_numpy(synth.make_blocks(fmt, N, K, seed=1)).cuda()
        Ws = [base] + [torch.roll(base, 1028160 * (i + 1)).contiguous() for i in range(R - 1)]
        X = torch.from_numpy(synth.make_activations(1, K, seed=2)).cuda()
        Y = torch.empty((1, N), dtype=torch.float32, device="cuda")
        buf = torch.zeros((n_launch, 160, 16), dtype=torch.int64, device="cuda")
        L.b200q_trace_set(None, 0)
        for i in range(3):
            ops.gemv(fmt, Ws[i % R], X, N, out=Y)
        torch.cuda.synchronize()
        L.b200q_trace_set(buf.data_ptr(), n_launch)
        g, st = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.graph(g, stream=st):
            for i in range(n_launch):
                ops.gemv(fmt, Ws[i % R], X, N, out=Y)
        L.b200q_trace_set(None, 0)
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); g.replay(); e1.record(); torch.cuda.synchronize()
        t = buf.cpu().numpy().astype(np.int64)
        acc = {}
        for i in range(4, n_launch - 1):
            c = t[i][t[i][:, 0] > 0]
            pv = t[i - 1][t[i - 1][:, 0] > 0]
            pend = max(pv[:, 5].max(), pv[:, 6].max())
            end = np.maximum(c[:, 5], c[:, 6])
            for k, v in (("ctas", len(c)), ("period", end.max() - pend), ("entry", np.median(c[:, 0] - pend)),
                         ("barriers_ready", np.median(c[:, 1] - pend)), ("first_copy_issued", np.median(c[:, 7] - pend)),
                         ("predecessor_complete", np.median(c[:, 2] - pend)), ("x_staged", np.median(c[:, 3] - pend)),
                         ("first_tile_started", np.median(c[:, 4] - pend)), ("last_copy_issued", np.median(c[:, 8] - pend)),
                         ("cta_end_median", np.median(end - pend)), ("cta_end_last", end.max() - pend)):
                acc.setdefault(k, []).append(float(v))
            for j in range(9, 16):  # activation-resident kernel: end of warp 0's items
                if (c[:, j] > 0).any():
                    acc.setdefault(f"warp0_item{j - 9}_done", []).append(float(np.median(c[:, j][c[:, j] > 0] - pend)))
        row = {"shape": f"{fname} {N}x{K} M=1", "us_per_launch_under_trace": round(e0.elapsed_time(e1) / n_launch * 1e3, 2)}
        row.update({k: round(float(np.median(v))) for k, v in acc.items()})
        rows.append(row)
        print(json.dumps(row), flush=True)
    print("device status", ops.device_status())


# --------------------------------------------------------------------------- GPU arm

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--replicas", type=int, default=8)
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--case", default=None, metavar="OP:FMT:N:K:M",
                    help="profiling driver: a handful of launches of one shape (op gemv|gemm|dequant, fmt q4k|q6k|q8_0) and nothing else")
    ap.add_argument("--launches", type=int, default=4, help="launches of --case")
    ap.add_argument("--opt", action="append", default=[], metavar="KEY=VALUE",
                    help="library option for --case / --phases (b200q_set_option), e.g. gemv_xr=0 for the tile kernel")
    ap.add_argument("--no-pdl", action="store_true", help="--phases without programmatic dependent launch")
    ap.add_argument("--phases", nargs="?", const="", default=None, metavar="FMT:N:K,...",
                    help="phase breakdown of the decode GEMV from %%globaltimer stamps (needs the trace build: "
                         "python -m brotensor_b200.build --trace; B200Q_LIB=brotensor_b200/lib/libb200q_trace.so)")
    args = ap.parse_args()
    if args.opt:
        from brotensor_b200 import ops as _ops
        for kv in args.opt:
            key, val = kv.split("=")
            _ops.set_option(key, int(val))
    if args.case:
        return run_case(args.case, args.launches)
    if args.phases is not None:
        return run_phases(0 if args.no_pdl else 1, *([args.phases] if args.phases else []))

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    layer_bytes = sum(synth.packed_bytes(f, n, k) for _, f, n, k in synth.LLAMA3_8B_LAYER_SET)
    config = {"workload": WORKLOAD, "gemvs_per_step": 7, "M": 1, "packed_weight_bytes_per_step": layer_bytes,
              "l2": f"graph rotates over {args.replicas} weight replicas ({args.replicas * layer_bytes >> 20} MiB >> 126 MiB L2)"}

    if args.impl == "reference":
        if rank != 0:
            return
        cb, k, w, ms = run_cpu_arm("reference", args.steps, max(args.warmup, 0))
        ref_cuda = None
        if not args.no_extras:
            # same-box comparator: the reference's own CUDA kernels recompiled for sm_100a (informational;
            # the line's value stays the CPU number, as the reference's path for this metric is its CPU code)
            try:
                import torch
                if torch.cuda.is_available():
                    import bench_extras
                    ref_cuda = bench_extras.reference_cuda(measured_peaks(), torch.cuda.current_stream(), ROOT)
                else:
                    ref_cuda = {"unavailable": "no CUDA device"}
            except Exception as e:  # noqa: BLE001 - the CPU line must still print
                ref_cuda = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        print(json.dumps({
            "impl": "reference", "metric": "q4k_q6k_decode_gemv_packed_weight_GBps", "value": cb["value"],
            "unit": "GB/s", "n_gpus": args.gpus, "steps": k, "warmup": w, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config, "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0, "reference_cuda_sm100a": ref_cuda}))
        return

    import torch
    import torch.distributed as dist
    from brotensor_b200 import ops

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    K_steps, W_steps, R = args.steps, max(args.warmup, 3), args.replicas
    peaks = measured_peaks()
    # Programmatic dependent launch: a GEMV's weight prefetch may start while the previous
    # kernel of the stream drains (its activations are still read only after that kernel
    # has completed). Legal here because no kernel in the timed stream writes weights.
    ops.set_option("pdl", 1)

    # ---- resident inputs: R replicas of the layer set (distinct seeds), activations per layer
    t_setup = time.time()
    host_layers = [synth.make_blocks(fmt, N, K, seed=100 + i + 1000 * rank)
                   for i, (_, fmt, N, K) in enumerate(synth.LLAMA3_8B_LAYER_SET)]
    replicas = []
    for r in range(R):
        rep = []
        for W in host_layers:
            t = torch.from_numpy(W).cuda()
            if r:  # cheap decorrelation of replica contents, layout and statistics unchanged
                t = torch.roll(t, shifts=r * 144 * 210 * 34)
            rep.append(t.contiguous())
        replicas.append(rep)
    acts_h = [synth.make_activations(1, K, seed=100 + i) for i, (_, _, _, K) in enumerate(synth.LLAMA3_8B_LAYER_SET)]
    acts = [torch.from_numpy(a).cuda() for a in acts_h]
    outs = [torch.empty((1, N), dtype=torch.float32, device="cuda") for _, _, N, _ in synth.LLAMA3_8B_LAYER_SET]

    def step(r):
        for (name, fmt, N, K), W, x, y in zip(synth.LLAMA3_8B_LAYER_SET, replicas[r % R], acts, outs):
            ops.gemv(fmt, W, x, N, out=y)

    # parity gate on this rank's inputs before anything is timed
    import oracle
    step(0)
    torch.cuda.synchronize()
    cpu = oracle.cpu()
    worst = 0.0
    for (name, fmt, N, K), Wh, xh, y in zip(synth.LLAMA3_8B_LAYER_SET, host_layers, acts_h, outs):
        if rank == 0 and name in ("k_proj", "o_proj", "down_proj"):
            worst = max(worst, oracle.rel_l2(y.cpu().numpy(), cpu.matmul(fmt, Wh, xh, threads=os.cpu_count() or 1)))
    assert worst < 2e-3, f"parity gate failed: rel-L2 {worst}"

    for i in range(W_steps):
        step(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    cap_stream = torch.cuda.Stream()
    with torch.cuda.graph(g, stream=cap_stream):
        for i in range(K_steps):
            step(i)
    g.replay()  # one untimed replay settles the graph upload
    torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # The K-step graph is replayed until the timed region covers at least 0.3 s (a single replay is
    # a few milliseconds: too short for the clock sampler and for a stable median); every replay is
    # timed on its own with CUDA events, the reported time is the median, the minimum goes along.
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    one_ms = max(e0.elapsed_time(e1), 1e-3)
    reps = int(min(400, max(5, 300.0 / one_ms + 1)))
    t = torch.tensor([float(reps)], device="cuda")
    if world > 1:  # the same number of replays on every rank
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    reps = int(t.item())
    times = []
    for _ in range(reps):
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms_total = float(np.median(times))
    ms_min = float(np.min(times))
    config["timed_region"] = f"{reps} replays of the {K_steps}-step graph, {sum(times) / 1e3:.2f} s in all; median per replay reported"
    t = torch.tensor([ms_total], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    ms_per_step = ms_total / K_steps
    value = world * layer_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- roofline of the dominant kernel: Q4_K streaming GEMV on the gate/up shape, timed alone
    _, fmt_d, N_d, K_d = synth.LLAMA3_8B_LAYER_SET[4]
    alg_bytes = synth.packed_bytes(fmt_d, N_d, K_d) + 4 * K_d + 4 * N_d
    gd = torch.cuda.CUDAGraph()
    n_dom = 64
    with torch.cuda.graph(gd, stream=cap_stream):
        for i in range(n_dom):
            ops.gemv(fmt_d, replicas[i % R][4 + (i // R) % 2], acts[4], N_d, out=outs[4])
    gd.replay()
    torch.cuda.synchronize()
    dts = []
    for _ in range(10):
        e0.record()
        gd.replay()
        e1.record()
        torch.cuda.synchronize()
        dts.append(e0.elapsed_time(e1) / n_dom)
    dom_ms = float(np.median(dts))
    achieved = alg_bytes / (dom_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "gemv_xr_q4k_kernel (activation-resident Q4_K decode GEMV) on 14336x4096 (gate_proj / up_proj)", "achieved": achieved,
                "peak": peaks["hbm_gbs"], "peak_source": peaks["source"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": DOMINANT_KERNEL_DRAM_TRAFFIC,
                "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch",
                "algorithmic_bytes_per_launch": alg_bytes,
                "us_per_launch": dom_ms * 1e3}

    # ---- e2e: host buffers through the C++ plugin (Tensor / dispatch / public ops) every step
    from brotensor_b200 import hostapi
    hostapi.init()
    e2e_R = min(R, 4)  # weight replicas owned by the host layer, rotated like the device-side ones
    h_weights = [[hostapi.Weight(fmt, W if r == 0 else np.roll(W, r * 144 * 210 * 34), N, K, local_rank)
                  for (_, fmt, N, K), W in zip(synth.LLAMA3_8B_LAYER_SET, host_layers)] for r in range(e2e_R)]
    sessions = [[hostapi.Session(w, 1, 0, 0) for w in rep] for rep in h_weights]

    # page-locked host arenas: the step's inputs and results live on the host, one buffer each
    layers = [hostapi.LayerSet(rep) for rep in h_weights]
    L0 = layers[0]
    x_arena = torch.zeros(L0.x_bytes, dtype=torch.uint8).pin_memory()
    y_arena = torch.zeros(L0.y_bytes, dtype=torch.uint8).pin_memory()
    for off, a in zip(L0.x_off, acts_h):
        x_arena[off:off + a.nbytes] = torch.from_numpy(a.reshape(-1).view(np.uint8))

    def e2e_enqueue(r):
        # host x arena -> device (one copy), the seven linear_forward_*_fp16 through the dispatcher,
        # device y arena -> host (one copy)
        layers[r % e2e_R].enqueue(x_arena.data_ptr(), y_arena.data_ptr())

    # The step is captured once per weight replica with the host layer's CudaGraphCapture (what
    # brotensor's decode loops do with its cuda_graph.h) and replayed: one launch and one
    # synchronisation per step; new inputs are written into the same pinned buffers.
    for r in range(e2e_R):
        e2e_enqueue(r)
    hostapi.sync(local_rank)
    graphs = []
    for r in range(e2e_R):
        with hostapi.Graph.capture() as gph:
            e2e_enqueue(r)
        graphs.append(gph)

    def e2e_step(r):
        graphs[r % e2e_R].launch()
        hostapi.sync(local_rank)

    def e2e_step_blocking(r):
        for sess, xh in zip(sessions[r % e2e_R], acts_h):
            sess.run(xh)  # brotensor-style blocking round trip per op (pageable host memory)

    def time_e2e(fn):
        for i in range(W_steps):
            fn(i)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(K_steps):
            fn(i)
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) * 1e3 / K_steps
        t = torch.tensor([ms], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    e2e_ms = time_e2e(e2e_step)
    e2e_blocking_ms = time_e2e(e2e_step_blocking)
    h2d, d2h = int(L0.x_bytes), int(L0.y_bytes)  # the two arena copies of a step
    e2e = {"value": world * layer_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "path": "brotensor_b200 C++ host layer: one Tensor::copy_raw_from_host_async of the pinned activation arena -> "
                   "seven linear_forward_*_fp16 through the dispatcher -> one copy_raw_to_host_async of the result arena, "
                   "captured once with CudaGraphCapture; one CudaGraph::launch and one sync per step",
           "blocking_per_op": {"value": world * layer_bytes / (e2e_blocking_ms * 1e-3) / 1e9, "ms_per_step": e2e_blocking_ms,
                               "path": "Tensor::from_raw_bytes_on -> op -> copy_to_host, blocking like brotensor's own round trips"},
           "note": "weights stay resident (model state); activations and results cross PCIe every step"}
    if rank == 0:  # the end-to-end path returns the oracle's answer too
        e2e_step(0)
        _, kfmt, kN, kK = synth.LLAMA3_8B_LAYER_SET[1]
        y1 = y_arena[L0.y_off[1]:L0.y_off[1] + 4 * kN].numpy().view(np.float32)
        err = oracle.rel_l2(y1.reshape(1, -1), cpu.matmul(kfmt, host_layers[1], acts_h[1], threads=os.cpu_count() or 1))
        assert err < 2e-3, f"end-to-end parity failed: rel-L2 {err}"
    assert ops.device_status() == 0

    extras = {}
    if not args.no_extras:
        try:
            import bench_extras
            extras = bench_extras.run(rank, world, peaks, cap_stream)
        except Exception as ex:  # extras never take the headline down
            extras = {"error": repr(ex)}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_baseline, _, _, _ = run_cpu_arm("port", 10, 1, budget_s=12.0)

    if rank == 0:
        print(json.dumps({
            "metric": "q4k_q6k_decode_gemv_packed_weight_GBps", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": K_steps, "warmup": W_steps, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
            "frac_of_hbm_peak": value / world / peaks["hbm_gbs"], "roofline": roofline, "cpu_baseline": cpu_baseline,
            "ms_per_step_min": ms_min / K_steps, "lm_head": lm_head_summary(extras, world),
            "e2e": e2e, "gpu_launches": 7 * K_steps, "clocks": clocks, "extras": extras,
            "setup_s": round(time.time() - t_setup, 1)}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

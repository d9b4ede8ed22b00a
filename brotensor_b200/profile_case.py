"""Runs a handful of launches of one decode-GEMV / prefill-GEMM shape, for profilers.

    python -m brotensor_b200.profile_case <fmt q4k|q6k|q8_0> <N> <K> <M> [--launches 4] [--path 0] [--op gemv|gemm|dequant]

The weights rotate over six replicas so that a captured launch streams from DRAM; the
device holds a few hundred MB at most. Prints the device status word at the end.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from brotensor_b200 import ops, synth  # noqa: E402

FMT = {"q4k": synth.Q4_K, "q6k": synth.Q6_K, "q8_0": synth.Q8_0}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("fmt", choices=sorted(FMT))
    ap.add_argument("N", type=int)
    ap.add_argument("K", type=int)
    ap.add_argument("M", type=int)
    ap.add_argument("--launches", type=int, default=4)
    ap.add_argument("--path", type=int, default=0)
    ap.add_argument("--op", default="gemv", choices=["gemv", "gemm", "dequant"])
    ap.add_argument("--replicas", type=int, default=6)
    a = ap.parse_args()
    fmt = FMT[a.fmt]
    torch.cuda.set_device(0)
    ops.set_option("gemv_path", a.path)
    base = torch.from_numpy(synth.make_blocks(fmt, a.N, a.K, seed=1)).cuda()
    Ws = [base] + [torch.roll(base, 1028160 * (i + 1)).contiguous() for i in range(a.replicas - 1)]
    X = torch.from_numpy(synth.make_activations(a.M, a.K, seed=2)).cuda()
    Y = torch.empty((a.M, a.N), dtype=torch.float32, device="cuda")
    if a.op == "dequant":  # decode to FP16 (M is ignored); the outputs rotate as well
        for i in range(a.launches):
            ops.dequant(fmt, Ws[i % len(Ws)], a.N, a.K, torch.float16)
        torch.cuda.synchronize()
        print("device status", ops.device_status())
        return
    f = ops.gemv if a.op == "gemv" else ops.gemm
    for i in range(a.launches):
        f(fmt, Ws[i % len(Ws)], X, a.N, out=Y)
    torch.cuda.synchronize()
    print("device status", ops.device_status())


if __name__ == "__main__":
    main()

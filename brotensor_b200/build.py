"""Builds the in-tree native libraries with nvcc for sm_100a.

    python -m brotensor_b200.build            # everything that is out of date
    python -m brotensor_b200.build --force

libb200q.so        the CUDA kernels behind the C-ABI of include/b200q.h
libbrotensor_b200.so  the C++20 host layer (Tensor / dispatch / GGUF loader / ops)
"""
from __future__ import annotations

import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
HOST = os.path.join(PKG, "host")
LIBDIR = os.path.join(PKG, "lib")
OBJDIR = os.path.join(PKG, "build")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH + ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "--use_fast_math=false"]
NVCC_FLAGS = [f for f in NVCC_FLAGS if f != "--use_fast_math=false"]

KERNEL_SOURCES = ["api.cu", "dequant.cu", "repack.cu", "gemv_simple.cu", "gemv_stream.cu", "gemv_dp.cu", "gemv_xr.cu", "gemv_i8.cu", "gemm_tc.cu", "gemm_tc2.cu", "gemm_static.cu"]


def _newer(src_list, target) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in src_list)


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("build step failed: " + " ".join(cmd[:3]))
    return r.stdout + r.stderr


def build_kernels(force: bool = False, verbose: bool = False, trace: bool = False) -> str:
    """libb200q.so; with `trace`, libb200q_trace.so: the same sources with -DB200Q_TRACE, whose decode GEMV
    stamps %globaltimer at the phases of a launch (read by `bench.py --phases`)."""
    os.makedirs(LIBDIR, exist_ok=True)
    objdir = os.path.join(OBJDIR, "trace") if trace else OBJDIR
    os.makedirs(objdir, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(ROOT, "include", "b200q.h"))
    objs = []
    procs = []
    for src in KERNEL_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(objdir, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _newer([s] + headers, o):
            cmd = [NVCC] + NVCC_FLAGS + (["-DB200Q_TRACE"] if trace else []) + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + out)
            raise RuntimeError("nvcc failed on " + cmd[-3])
        if verbose:
            sys.stderr.write(out)
    lib = os.path.join(LIBDIR, "libb200q_trace.so" if trace else "libb200q.so")
    if force or procs or _newer(objs, lib):
        _run([NVCC] + ARCH + ["-shared", "-o", lib] + objs + ["-lcudart"])
    return lib


def build_host(force: bool = False) -> str | None:
    """C++20 host layer; links against libb200q.so."""
    if not os.path.isdir(HOST):
        return None
    srcs = sorted(os.path.join(HOST, f) for f in os.listdir(HOST) if f.endswith(".cpp"))
    if not srcs:
        return None
    hdrs = []
    for d, _, fs in os.walk(os.path.join(ROOT, "include")):
        hdrs += [os.path.join(d, f) for f in fs]
    lib = os.path.join(LIBDIR, "libbrotensor_b200.so")
    if force or _newer(srcs + hdrs, lib):
        _run(["g++", "-std=c++20", "-O2", "-fPIC", "-shared", "-Wall", "-o", lib] + srcs +
             ["-I" + os.path.join(ROOT, "include"), "-I/usr/local/cuda/include", "-L" + LIBDIR, "-lb200q",
              "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,$ORIGIN", "-lpthread"])
    return lib


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force, verbose)
    build_host(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    if "--trace" in sys.argv:
        build_kernels(force="--force" in sys.argv, trace=True)
    print("built:", ", ".join(sorted(os.listdir(LIBDIR))))

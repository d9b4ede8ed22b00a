"""Builds the C++ test executable of the host layer (tests/cpp/host_tests.cpp -> tests/cpp/host_tests).

Test infrastructure: it links the product libraries (brotensor_b200/lib) and the CPU oracle as its
checker. The product build (brotensor_b200.build) knows nothing about it.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
LIBDIR = os.path.join(ROOT, "brotensor_b200", "lib")
ORACLE = os.path.join(ROOT, "oracle")
EXE = os.path.join(HERE, "host_tests")


def build(force: bool = False) -> str:
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    from brotensor_b200 import build as product
    product.build_all()
    subprocess.run(["make", "-s", "-C", ORACLE, os.path.join(ORACLE, "liboracle.so")], check=True)
    src = os.path.join(HERE, "host_tests.cpp")
    deps = [src, os.path.join(LIBDIR, "libbrotensor_b200.so"), os.path.join(ORACLE, "liboracle.so")]
    if force or not os.path.exists(EXE) or any(os.path.getmtime(d) > os.path.getmtime(EXE) for d in deps):
        cmd = ["g++", "-std=c++20", "-O1", "-o", EXE, src, "-I" + os.path.join(ROOT, "include"), "-I/usr/local/cuda/include",
               "-L" + LIBDIR, "-lbrotensor_b200", "-lb200q", "-L" + ORACLE, "-loracle", "-L/usr/local/cuda/lib64", "-lcudart",
               "-Wl,-rpath," + LIBDIR, "-Wl,-rpath," + ORACLE, "-lpthread"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            raise RuntimeError("building tests/cpp/host_tests failed")
    return EXE


if __name__ == "__main__":
    print(build("--force" in sys.argv))

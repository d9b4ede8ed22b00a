"""brotensor_b200 — B200 (sm_100a) GGUF fused quant-matmul backend.

Python here is harness only (tests, benchmark, multi-GPU launch): it hands
device pointers of torch tensors to the C-ABI in include/b200q.h. All compute
is in the CUDA library; importing the ops without the built library raises.
"""
from . import synth  # noqa: F401
from ._capi import B200QError, BF16, F16, F32, Q4_K, Q6_K, Q8_0  # noqa: F401

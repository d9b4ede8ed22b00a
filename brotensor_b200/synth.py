"""Seeded synthetic GGUF blocks and activations with the shapes, sizes and value
distributions of the benchmark configurations (they stand in for a Llama-3-8B
GGUF file; no model content is involved).

Block layouts follow the reference's device structs: Q4_K
src/cuda/q4k_internal.cuh:4-9, Q6_K src/cuda/q6k_internal.cuh:5-9, Q8_0
src/cuda/q8_0_internal.cuh:13-16. Pure numpy; used by the benchmark and tests.
"""
from __future__ import annotations

import numpy as np

Q8_0, Q4_K, Q6_K = 14, 22, 24
Q4_0, Q5_K = 10, 23  # ggml block_q4_0 / block_q5_K
Q6_K_R8 = 124  # device-side regrouped form of Q6_K (same bytes per block; see include/b200q.h)
BLOCK_ELEMS = {Q8_0: 32, Q4_K: 256, Q6_K: 256, Q6_K_R8: 256, Q4_0: 32, Q5_K: 256}
BLOCK_BYTES = {Q8_0: 34, Q4_K: 144, Q6_K: 210, Q6_K_R8: 210, Q4_0: 18, Q5_K: 176}
FMT_NAME = {Q8_0: "q8_0", Q4_K: "q4k", Q6_K: "q6k", Q6_K_R8: "q6k_r8", Q4_0: "q4_0", Q5_K: "q5k"}


def packed_bytes(fmt: int, rows: int, K: int) -> int:
    assert K % BLOCK_ELEMS[fmt] == 0
    return rows * (K // BLOCK_ELEMS[fmt]) * BLOCK_BYTES[fmt]


def _f16_bytes(rng: np.random.Generator, n: int, scale: float) -> np.ndarray:
    v = (np.abs(rng.standard_normal(n, dtype=np.float32)) * np.float32(scale)).astype(np.float16)
    return v.view(np.uint8).reshape(n, 2)


def make_blocks(fmt: int, rows: int, K: int, seed: int) -> np.ndarray:
    """Row-major [rows][K/elems][block bytes] as a flat uint8 array.

    Q4_K: d, dmin = fp16(|N(0,1)|*0.002); 12 uniform bytes = eight 6-bit scales and
    eight 6-bit mins uniform in 0..63 under the 6-bit packing (a bijection on 96
    bits); 128 uniform bytes of 4-bit quants.
    Q6_K: 128 + 64 uniform bytes, 16 int8 sub-scales uniform in -32..31,
    d = fp16(|N(0,1)|*0.001).
    Q8_0: d = fp16(|N(0,1)|*0.005), 32 int8 uniform in -127..127.
    """
    rng = np.random.default_rng(np.random.PCG64(seed))
    nb = rows * (K // BLOCK_ELEMS[fmt])
    out = np.empty((nb, BLOCK_BYTES[fmt]), np.uint8)
    if fmt == Q4_K:
        out[:, 0:2] = _f16_bytes(rng, nb, 0.002)
        out[:, 2:4] = _f16_bytes(rng, nb, 0.002)
        out[:, 4:144] = rng.integers(0, 256, size=(nb, 140), dtype=np.uint8)
    elif fmt == Q6_K:
        out[:, 0:192] = rng.integers(0, 256, size=(nb, 192), dtype=np.uint8)
        out[:, 192:208] = rng.integers(-32, 32, size=(nb, 16), dtype=np.int8).view(np.uint8)
        out[:, 208:210] = _f16_bytes(rng, nb, 0.001)
    elif fmt == Q8_0:
        out[:, 0:2] = _f16_bytes(rng, nb, 0.005)
        out[:, 2:34] = rng.integers(-127, 128, size=(nb, 32), dtype=np.int8).view(np.uint8)
    elif fmt == Q4_0:  # d = fp16(|N(0,1)|*0.005), 16 uniform bytes of 4-bit quants
        out[:, 0:2] = _f16_bytes(rng, nb, 0.005)
        out[:, 2:18] = rng.integers(0, 256, size=(nb, 16), dtype=np.uint8)
    elif fmt == Q5_K:  # as Q4_K plus 32 uniform bytes of fifth bits
        out[:, 0:2] = _f16_bytes(rng, nb, 0.002)
        out[:, 2:4] = _f16_bytes(rng, nb, 0.002)
        out[:, 4:176] = rng.integers(0, 256, size=(nb, 172), dtype=np.uint8)
    else:
        raise ValueError(f"unknown block format {fmt}")
    return out.reshape(-1)


def make_activations(M: int, K: int, seed: int) -> np.ndarray:
    """(M, K) fp32 drawn N(0,1) from a stream separate from the weight stream."""
    rng = np.random.default_rng(np.random.PCG64(seed + 0x9E3779B9))
    return rng.standard_normal((M, K), dtype=np.float32)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit patterns, round to nearest even."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + (0x7FFF + ((u >> 16) & 1))) >> 16).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


# The Llama-3-8B-shaped decode layer set: (name, format, N, K).
LLAMA3_8B_LAYER_SET = [
    ("q_proj", Q4_K, 4096, 4096),
    ("k_proj", Q4_K, 1024, 4096),
    ("v_proj", Q4_K, 1024, 4096),
    ("o_proj", Q4_K, 4096, 4096),
    ("gate_proj", Q4_K, 14336, 4096),
    ("up_proj", Q4_K, 14336, 4096),
    ("down_proj", Q6_K, 4096, 14336),
]

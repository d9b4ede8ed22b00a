// Shared device/host helpers of the b200q kernels: block-format traits, exact
// scalar decode of the three GGUF block formats, small PTX wrappers (mbarrier,
// bulk async copy, warp MMA) and the host-side error plumbing.
//
// Block layouts (GGUF), as brotensor's device structs define them:
//   Q4_K  src/cuda/q4k_internal.cuh:4-9   144 B: fp16 d @0, fp16 dmin @2, u8 scales[12] @4, u8 qs[128] @16
//   Q6_K  src/cuda/q6k_internal.cuh:5-9   210 B: u8 ql[128] @0, u8 qh[64] @128, i8 scales[16] @192, fp16 d @208
//   Q8_0  src/cuda/q8_0_internal.cuh:13-16 34 B: fp16 d @0, i8 qs[32] @2
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200q.h"

namespace b200q {

constexpr int kQ8_0 = B200Q_FMT_Q8_0;
constexpr int kQ4_K = B200Q_FMT_Q4_K;
constexpr int kQ6_K = B200Q_FMT_Q6_K;
constexpr int kQ6_KP = B200Q_FMT_Q6_K_R8;  // Q6_K regrouped by field in runs of eight blocks
constexpr int kQ4_0 = B200Q_FMT_Q4_0;
constexpr int kQ5_K = B200Q_FMT_Q5_K;
constexpr int kQ6RunBytes = 1680, kQ6RunElems = 2048;

// Device status codes written by kernels whose bounded waits run out.
constexpr int kDevTimeoutFull = 101;   // consumer gave up waiting for a filled stage
constexpr int kDevTimeoutEmpty = 102;  // producer gave up waiting for a free stage
constexpr int kDevTimeoutMma = 103;    // epilogue gave up waiting for the tensor core
constexpr int kDevTimeoutTmem = 104;
constexpr int kDevTimeoutPeer = 105;   // sharded GEMV gave up waiting for a peer rank's arrival flag

template <int FMT>
struct Blk;
template <>
struct Blk<kQ4_K> {
    static constexpr int elems = 256, bytes = 144, align = 4;
    // smallest run of blocks whose byte length is a multiple of 16 (bulk-copy granule)
    static constexpr int chunk_blocks = 1;
};
template <>
struct Blk<kQ6_K> {
    static constexpr int elems = 256, bytes = 210, align = 2;
    static constexpr int chunk_blocks = 8;
};
template <>
struct Blk<kQ6_KP> {  // per block the same 210 bytes; addressable only in whole runs of eight
    static constexpr int elems = 256, bytes = 210, align = 16;
    static constexpr int chunk_blocks = 8;
};
template <>
struct Blk<kQ8_0> {
    static constexpr int elems = 32, bytes = 34, align = 2;
    static constexpr int chunk_blocks = 8;
};
template <>
struct Blk<kQ4_0> {  // ggml block_q4_0
    static constexpr int elems = 32, bytes = 18, align = 2;
    static constexpr int chunk_blocks = 8;
};
template <>
struct Blk<kQ5_K> {  // ggml block_q5_K
    static constexpr int elems = 256, bytes = 176, align = 4;
    static constexpr int chunk_blocks = 1;
};

// ---- host-side error plumbing ------------------------------------------------
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);

constexpr int kMaxShardRanks = 8;
constexpr int kMaxTopK = 8;      // candidates per CTA in the candidate form of the sharded head
constexpr int kShardSlots = 256;  // CTA slots per rank in a candidate table (an upper bound of the grid)
constexpr int kMaxSegments = 4;  // weight matrices one grouped GEMV launch can take
// Host-side description of a row-sharded GEMV output (StreamParams::sh_* on the device side).
struct ShardOut {
    int world, rank, row_offset, total_rows;
    float* const* out;
    unsigned int* state;
    // candidate form: k in 1..kMaxTopK, every rank's candidate table, this rank's results (else 0 / null)
    int topk = 0;
    uint32_t* const* cand = nullptr;
    float* top_val = nullptr;
    int* top_idx = nullptr;
};
int* device_status_word(int dev);  // device pointer to this device's status word, or nullptr

#define B200Q_CUDA_TRY(expr)                                                                          \
    do {                                                                                              \
        cudaError_t e_ = (expr);                                                                      \
        if (e_ != cudaSuccess && (cudaGetLastError(), true)) /* report once, leave no sticky error */ \
            return ::b200q::fail(B200Q_ERR_CUDA, "CUDA error %d (%s) at %s:%d in `%s`", (int)e_,      \
                                 cudaGetErrorString(e_), __FILE__, __LINE__, #expr);                  \
    } while (0)

#ifdef __CUDACC__
// ---- raw loads at the alignment the formats guarantee -------------------------
__device__ __forceinline__ uint32_t ld_nc_u32(const void* p) { return __ldg(reinterpret_cast<const unsigned int*>(p)); }
__device__ __forceinline__ uint32_t ld_nc_u16(const void* p) {
    return __ldg(reinterpret_cast<const unsigned short*>(p));
}
// 4 bytes from an address that is only 2-byte aligned.
__device__ __forceinline__ uint32_t ld_nc_u32_a2(const uint8_t* p) { return ld_nc_u16(p) | (ld_nc_u16(p + 2) << 16); }
template <int ALIGN>
__device__ __forceinline__ uint32_t ld_w(const uint8_t* p) {
    if constexpr (ALIGN >= 4) return ld_nc_u32(p);
    else return ld_nc_u32_a2(p);
}
__device__ __forceinline__ float h2f(uint32_t bits16) { return __half2float(__ushort_as_half((unsigned short)bits16)); }

// ---- exact decode of 8 consecutive elements -----------------------------------
// `row` points at the first block of a weight row; `u` indexes groups of eight
// consecutive elements along the row. Every product below is exact in FP32 and
// the single subtraction rounds the exact value, so the result is independent of
// operation order and FMA contraction.
template <int FMT>
__device__ __forceinline__ void decode8(const uint8_t* __restrict__ row, int u, float w[8]);

template <>
__device__ __forceinline__ void decode8<kQ4_K>(const uint8_t* __restrict__ row, int u, float w[8]) {
    const uint8_t* blk = row + (size_t)(u >> 5) * 144;
    const int i = u & 31, is = i >> 2, l0 = (i & 3) * 8;
    const uint32_t dd = ld_nc_u32(blk);
    const uint32_t s0 = ld_nc_u32(blk + 4), s1 = ld_nc_u32(blk + 8), s2 = ld_nc_u32(blk + 12);
    uint32_t sc, m;
    if (is < 4) {
        sc = (s0 >> (8 * is)) & 63u;
        m = (s1 >> (8 * is)) & 63u;
    } else {
        const int j = is - 4;
        sc = ((s2 >> (8 * j)) & 0xFu) | (((s0 >> (8 * j + 6)) & 3u) << 4);
        m = ((s2 >> (8 * j + 4)) & 0xFu) | (((s1 >> (8 * j + 6)) & 3u) << 4);
    }
    const float ds = h2f(dd & 0xFFFFu) * (float)sc;
    const float dm = h2f(dd >> 16) * (float)m;
    const uint8_t* q = blk + 16 + (is >> 1) * 32 + l0;
    uint32_t q0 = ld_nc_u32(q), q1 = ld_nc_u32(q + 4);
    if (is & 1) {
        q0 >>= 4;
        q1 >>= 4;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        w[k] = ds * (float)((q0 >> (8 * k)) & 0xFu) - dm;
        w[4 + k] = ds * (float)((q1 >> (8 * k)) & 0xFu) - dm;
    }
}

template <>
__device__ __forceinline__ void decode8<kQ6_K>(const uint8_t* __restrict__ row, int u, float w[8]) {
    const uint8_t* blk = row + (size_t)(u >> 5) * 210;
    const int i = u & 31, group = i >> 4, quad = (i & 15) >> 2, l0 = (i & 3) * 8;
    const int sb = group * 8 + quad * 2 + (l0 >> 4);
    const uint8_t* ql = blk + group * 64 + (quad & 1) * 32 + l0;
    const uint8_t* qh = blk + 128 + group * 32 + l0;
    uint32_t a0 = ld_nc_u32_a2(ql), a1 = ld_nc_u32_a2(ql + 4);
    const uint32_t h0 = ld_nc_u32_a2(qh) >> (quad * 2), h1 = ld_nc_u32_a2(qh + 4) >> (quad * 2);
    if (quad >= 2) {
        a0 >>= 4;
        a1 >>= 4;
    }
    const uint32_t scd = ld_nc_u16(blk + 192 + (sb & ~1));
    const int sc = (int)(signed char)((scd >> ((sb & 1) * 8)) & 0xFFu);
    const float ds = h2f(ld_nc_u16(blk + 208)) * (float)sc;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int v0 = (int)(((a0 >> (8 * k)) & 0xFu) | (((h0 >> (8 * k)) & 3u) << 4)) - 32;
        const int v1 = (int)(((a1 >> (8 * k)) & 0xFu) | (((h1 >> (8 * k)) & 3u) << 4)) - 32;
        w[k] = ds * (float)v0;
        w[4 + k] = ds * (float)v1;
    }
}

template <>
__device__ __forceinline__ void decode8<kQ6_KP>(const uint8_t* __restrict__ row, int u, float w[8]) {
    const int b = u >> 5;  // block along the row; run b >> 3, slot b & 7
    const uint8_t* run = row + (size_t)(b >> 3) * kQ6RunBytes;
    const int s = b & 7;
    const int i = u & 31, group = i >> 4, quad = (i & 15) >> 2, l0 = (i & 3) * 8;
    const int sb = group * 8 + quad * 2 + (l0 >> 4);
    const uint2 a = __ldg(reinterpret_cast<const uint2*>(run + s * 128 + group * 64 + (quad & 1) * 32 + l0));
    const uint2 h = __ldg(reinterpret_cast<const uint2*>(run + 1024 + s * 64 + group * 32 + l0));
    uint32_t a0 = a.x, a1 = a.y;
    const uint32_t h0 = h.x >> (quad * 2), h1 = h.y >> (quad * 2);
    if (quad >= 2) {
        a0 >>= 4;
        a1 >>= 4;
    }
    const int sc = (int)(signed char)__ldg(run + 1536 + s * 16 + sb);
    const float ds = h2f(ld_nc_u16(run + 1664 + 2 * s)) * (float)sc;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int v0 = (int)(((a0 >> (8 * k)) & 0xFu) | (((h0 >> (8 * k)) & 3u) << 4)) - 32;
        const int v1 = (int)(((a1 >> (8 * k)) & 0xFu) | (((h1 >> (8 * k)) & 3u) << 4)) - 32;
        w[k] = ds * (float)v0;
        w[4 + k] = ds * (float)v1;
    }
}

template <>
__device__ __forceinline__ void decode8<kQ8_0>(const uint8_t* __restrict__ row, int u, float w[8]) {
    const uint8_t* blk = row + (size_t)(u >> 2) * 34;
    const float d = h2f(ld_nc_u16(blk));
    const uint8_t* q = blk + 2 + (u & 3) * 8;
    const uint32_t q0 = ld_nc_u32_a2(q), q1 = ld_nc_u32_a2(q + 4);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        w[k] = d * (float)(int)(signed char)((q0 >> (8 * k)) & 0xFFu);
        w[4 + k] = d * (float)(int)(signed char)((q1 >> (8 * k)) & 0xFFu);
    }
}

// Q4_0 (ggml block_q4_0, dequantize_row_q4_0): element j of a block is the low nibble of qs[j] for
// j < 16 and the high nibble of qs[j - 16] otherwise, minus 8, times d. d * (q - 8): 11 + 4 bits, exact.
template <>
__device__ __forceinline__ void decode8<kQ4_0>(const uint8_t* __restrict__ row, int u, float w[8]) {
    const uint8_t* blk = row + (size_t)(u >> 2) * 18;
    const float d = h2f(ld_nc_u16(blk));
    const int part = u & 3;  // elements 8 * part .. 8 * part + 7
    const uint8_t* q = blk + 2 + (part & 1) * 8;
    uint32_t q0 = ld_nc_u32_a2(q), q1 = ld_nc_u32_a2(q + 4);
    if (part >= 2) {
        q0 >>= 4;
        q1 >>= 4;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        w[k] = d * (float)((int)((q0 >> (8 * k)) & 0xFu) - 8);
        w[4 + k] = d * (float)((int)((q1 >> (8 * k)) & 0xFu) - 8);
    }
}

// Q5_K (ggml block_q5_K, dequantize_row_q5_K): d @0, dmin @2, scales[12] @4 packed as in Q4_K, qh[32] @16,
// qs[128] @48. Sub-block is = 0..7 of 32 elements: byte qs[(is >> 1) * 32 + l], low nibble for even is,
// high nibble for odd; the fifth bit is bit `is` of qh[l]. w = d * sc * q - dmin * m with q in 0..31:
// 11 + 6 + 5 bits and 11 + 6 bits, both exact in FP32, one rounding in the subtraction.
template <>
__device__ __forceinline__ void decode8<kQ5_K>(const uint8_t* __restrict__ row, int u, float w[8]) {
    const uint8_t* blk = row + (size_t)(u >> 5) * 176;
    const int i = u & 31, is = i >> 2, l0 = (i & 3) * 8;
    const uint32_t dd = ld_nc_u32(blk);
    const uint32_t s0 = ld_nc_u32(blk + 4), s1 = ld_nc_u32(blk + 8), s2 = ld_nc_u32(blk + 12);
    uint32_t sc, m;
    if (is < 4) {
        sc = (s0 >> (8 * is)) & 63u;
        m = (s1 >> (8 * is)) & 63u;
    } else {
        const int j = is - 4;
        sc = ((s2 >> (8 * j)) & 0xFu) | (((s0 >> (8 * j + 6)) & 3u) << 4);
        m = ((s2 >> (8 * j + 4)) & 0xFu) | (((s1 >> (8 * j + 6)) & 3u) << 4);
    }
    const float ds = h2f(dd & 0xFFFFu) * (float)sc;
    const float dm = h2f(dd >> 16) * (float)m;
    const uint8_t* q = blk + 48 + (is >> 1) * 32 + l0;
    const uint8_t* h = blk + 16 + l0;
    uint32_t q0 = ld_nc_u32(q), q1 = ld_nc_u32(q + 4);
    const uint32_t h0 = ld_nc_u32(h) >> is, h1 = ld_nc_u32(h + 4) >> is;
    if (is & 1) {
        q0 >>= 4;
        q1 >>= 4;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        w[k] = ds * (float)(((q0 >> (8 * k)) & 0xFu) | (((h0 >> (8 * k)) & 1u) << 4)) - dm;
        w[4 + k] = ds * (float)(((q1 >> (8 * k)) & 0xFu) | (((h1 >> (8 * k)) & 1u) << 4)) - dm;
    }
}

// ---- element type helpers -----------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ---- shared-memory addresses, mbarrier, bulk async copy -----------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking probe of a phase (try_wait may park the thread for a hardware time slice).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls (each poll itself blocks for a
// hardware-defined slice), records `code` in the device status word and returns
// false. Callers stop using the pipeline when it fails; nothing traps.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, int* status, int code,
                                                  uint32_t limit = (1u << 22)) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    if (status) atomicCAS(status, 0, code);
    return false;
}
// 1-D bulk copy global -> shared; both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- warp-level MMA (FP16 operands, FP32 accumulators) ------------------------
// D(16x8) += A(16x16) * B(16x8). Lane = 4*g + t holds
//   a0: (row g,   k 2t..2t+1)   a1: (row g+8, k 2t..2t+1)
//   a2: (row g,   k 2t+8..2t+9) a3: (row g+8, k 2t+8..2t+9)
//   b0: (k 2t..2t+1, col g)     b1: (k 2t+8..2t+9, col g)
//   c0,c1: (row g, cols 2t,2t+1) c2,c3: (row g+8, cols 2t,2t+1)
__device__ __forceinline__ void mma16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// D(16x8) += A(16x8) * B(8x8): a0: (row g, k 2t..2t+1), a1: (row g+8, same k), b0: (k 2t..2t+1, col g).
__device__ __forceinline__ void mma1688(float c[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a & mask) | orv
    return r;
}
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
// Shared-memory accesses with a compile-time byte offset folded into the instruction.
template <int IMM>
__device__ __forceinline__ uint4 lds128i(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr), "n"(IMM));
    return v;
}
template <int IMM>
__device__ __forceinline__ uint32_t lds32i(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(IMM));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
#endif  // __CUDACC__

}  // namespace b200q

// Pieces shared by the integer-dot-product decode GEMV kernels (gemv_dp.cu, gemv_xr.cu): the dp2a
// wrappers, the layout constant of the staged activations, the dtype-generic activation load and the
// Q4_K inner product of 64 quants.
#pragma once
#include "stream_common.cuh"

namespace b200q {

// Trace builds (-DB200Q_TRACE, `python -m brotensor_b200.build --trace`) stamp %globaltimer at the phases of a
// launch into slot k of the CTA's sixteen-word record; the product build carries none of it.
#ifdef B200Q_TRACE
#define TRACE_STAMP(cond, k)                                                               \
    do {                                                                                   \
        if (p.trace && (cond)) p.trace[(size_t)blockIdx.x * 16 + (k)] = global_timer_ns(); \
    } while (0)
#else
#define TRACE_STAMP(cond, k) \
    do {                     \
    } while (0)
#endif
#ifdef B200Q_TRACE
unsigned long long* dp_trace_next(int grid);
#endif

__device__ __forceinline__ int dp2a_lo_su(uint32_t x, uint32_t b, int c) {  // signed x pairs, unsigned bytes
    int d;
    asm("dp2a.lo.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(x), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp2a_hi_su(uint32_t x, uint32_t b, int c) {
    int d;
    asm("dp2a.hi.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(x), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp2a_lo_ss(uint32_t x, uint32_t b, int c) {  // signed x pairs, signed bytes
    int d;
    asm("dp2a.lo.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(x), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp2a_hi_ss(uint32_t x, uint32_t b, int c) {
    int d;
    asm("dp2a.hi.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(x), "r"(b), "r"(c));
    return d;
}

// Staged activations: group gg of row m is 16 segments of eight int16. Groups are laid
// out at a stride of 272 bytes (256 + 16), so lanes working on consecutive groups read
// the same segment number from consecutive 16-byte bank groups (conflict-free) and a
// segment's address is the group's base plus a compile-time offset. All shared-memory
// traffic below goes through explicit ld.shared / st.shared with 32-bit addresses.
constexpr int kXGroupStride = 272;

// Eight consecutive activations (segment `idx` of the M x K matrix) as floats, whatever the element
// type: the type is a run-time switch around the load alone, so that the staging code exists once
// per kernel instead of once per type (it used to be two thirds of the kernel's instructions, all of
// them fetched cold at every launch).
__device__ __forceinline__ void x_load_seg(const void* base, int x_dtype, int K, int idx, float (&v)[8]) {
    const int segs = K >> 3;
    const int m = idx / segs, seg = idx - m * segs;
    if (x_dtype == B200Q_DT_F32) {
        const float4* X = reinterpret_cast<const float4*>(static_cast<const float*>(base) + (size_t)m * K) + 2 * seg;
        const float4 a = __ldg(X), b = __ldg(X + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + (size_t)m * K) + seg);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        if (x_dtype == B200Q_DT_F16) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
                v[2 * k] = f.x;
                v[2 * k + 1] = f.y;
            }
        } else {  // BF16: the upper half of an FP32
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                v[2 * k] = __uint_as_float(w[k] << 16);
                v[2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
            }
        }
    }
}

// 32 bytes of quants (two uint4) against 64 activations: low nibbles pair with x[0..3],
// high nibbles (left in place, i.e. times 16) with x[4..7].
__device__ __forceinline__ void q4k_dot(const uint4& q0, const uint4& q1, const uint4 (&x)[8], int& cl, int& ch) {
    const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    // two independent chains per nibble set keep the integer pipe busy
    int a0 = 0, a1 = 0, b0 = 0, b1 = 0;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        const uint32_t l0 = w[2 * s] & 0x0F0F0F0Fu, l1 = w[2 * s + 1] & 0x0F0F0F0Fu;
        const uint32_t h0 = w[2 * s] & 0xF0F0F0F0u, h1 = w[2 * s + 1] & 0xF0F0F0F0u;
        a0 = dp2a_lo_su(x[s].x, l0, a0);
        a0 = dp2a_hi_su(x[s].y, l0, a0);
        a1 = dp2a_lo_su(x[s].z, l1, a1);
        a1 = dp2a_hi_su(x[s].w, l1, a1);
        b0 = dp2a_lo_su(x[4 + s].x, h0, b0);
        b0 = dp2a_hi_su(x[4 + s].y, h0, b0);
        b1 = dp2a_lo_su(x[4 + s].z, h1, b1);
        b1 = dp2a_hi_su(x[4 + s].w, h1, b1);
    }
    cl = a0 + a1;
    ch = (b0 + b1) >> 4;  // exact: every term is a multiple of 16
}

}  // namespace b200q

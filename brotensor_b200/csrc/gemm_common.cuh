// Pieces shared by the tensor-core prefill GEMM kernels (gemm_tc.cu: one CTA per 128 weight
// rows; gemm_tc2.cu: a CTA pair per 256 rows): launch parameters, the activation pre-pass,
// tcgen05 / TMEM wrappers, shared-memory and instruction descriptors, and the decode
// helpers that write the A operand.
#pragma once

#include "stream_common.cuh"

namespace b200q {

constexpr int kGemmRows = 128;           // weight rows per CTA (UMMA M)
constexpr int kBK = 64;                  // k per stage: one 128-byte swizzle row of FP16
constexpr int kMaxTokens = 512;          // per pass: two accumulators of 256 TMEM columns
constexpr int kGemmMaxStages = 6;

struct GemmParams {
    const uint8_t* W;
    const uint8_t* Xp;   // prepared activations of this pass: [K/64][tok_pad][64] FP16, swizzled rows
    const void* bias;    // N values of bias_dtype, or nullptr
    void* Y;             // first token row of this pass
    int* status;
    int tokens;          // valid tokens of this pass
    int tok_pad;         // tokens rounded up to 16 (N of the MMA; <= 512)
    int xp_tok_stride;   // rows per k-block in Xp (padded token count of the whole call)
    int N, K;
    int row_bytes;
    int bias_dtype, y_dtype;
    int n_stages;
    int stage_bytes;     // A (16 KB) + B (tok_pad * 128)
};

// ---- activation pre-pass ---------------------------------------------------------------
// Xp[kb][t][c ^ (t & 7)] (16-byte chunks) = FP16(X[t][64*kb + 8*c .. +8]); rows t >= M are zero.
template <typename XT>
__global__ void __launch_bounds__(256) gemm_xprep_kernel(const XT* __restrict__ X, uint4* __restrict__ Xp, int M,
                                                         int tok_pad, int K) {
    const long long total = (long long)(K / 64) * tok_pad * 8;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(idx & 7);
        const long long rowi = idx >> 3;  // kb * tok_pad + t
        const int t = (int)(rowi % tok_pad), kb = (int)(rowi / tok_pad);
        union {
            __half h[8];
            uint4 v;
        } o;
        if (t < M) {
            const XT* src = X + (size_t)t * K + (size_t)kb * 64 + c * 8;
            if constexpr (sizeof(XT) == 4) {
                const float4 a = __ldg(reinterpret_cast<const float4*>(src)), b = __ldg(reinterpret_cast<const float4*>(src) + 1);
                o.h[0] = __float2half_rn(a.x); o.h[1] = __float2half_rn(a.y); o.h[2] = __float2half_rn(a.z); o.h[3] = __float2half_rn(a.w);
                o.h[4] = __float2half_rn(b.x); o.h[5] = __float2half_rn(b.y); o.h[6] = __float2half_rn(b.z); o.h[7] = __float2half_rn(b.w);
            } else {
                union {
                    uint4 q;
                    XT e[8];
                } in;
                in.q = __ldg(reinterpret_cast<const uint4*>(src));
#pragma unroll
                for (int k = 0; k < 8; ++k) o.h[k] = __float2half_rn(to_f32<XT>(in.e[k]));
            }
        } else {
            o.v = make_uint4(0, 0, 0, 0);
        }
        Xp[rowi * 8 + (c ^ (t & 7))] = o.v;
    }
}

// ---- tcgen05 wrappers ---------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand tile, 128-byte swizzle, rows of 128 bytes in groups of eight (1024 bytes):
// start address >> 4, leading byte offset 1 (unused for swizzled K-major), stride byte
// offset 1024 >> 4, descriptor version 1 (sm_100), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16 instruction descriptor: D = F32, A = B = F16, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t instr_desc_f16(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kGemmRows >> 4) << 24);
}

// ---- A-operand producers: 64 weights of one row -> eight swizzled 16-byte chunks -----------
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// four nibble bytes (already masked to 0..15) -> w = ds * n - dm, exact in FP32, two half2 words
__device__ __forceinline__ void nib4_to_h2(uint32_t nib, float ds, float dm, uint32_t& o0, uint32_t& o1) {
    float f[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float n = __uint_as_float(__byte_perm(nib, 0x4B000000u, 0x7440 | i)) - 8388608.0f;  // exact 0..15
        f[i] = fmaf(ds, n, -dm);  // ds * n and dm are exact, one rounding: the reference's d*sc*nib - dmin*m
    }
    o0 = pack_h2(f[0], f[1]);
    o1 = pack_h2(f[2], f[3]);
}

// Pair P of a Q4_K block held in registers: low nibbles are sub-block 2P (k 0..31 of the
// stage), high nibbles sub-block 2P+1 (k 32..63).
template <int P>
__device__ __forceinline__ void q4k_pair_to_smem(const uint4 (&blk)[9], uint32_t rowaddr, uint32_t r7) {
    const uint4 h = blk[0];
    uint32_t sc0, sc1, m0, m1;
    if constexpr (P < 2) {
        sc0 = (h.y >> (16 * P)) & 63u; sc1 = (h.y >> (16 * P + 8)) & 63u;
        m0 = (h.z >> (16 * P)) & 63u;  m1 = (h.z >> (16 * P + 8)) & 63u;
    } else {
        constexpr int J = 2 * (P - 2);
        sc0 = ((h.w >> (8 * J)) & 0xFu) | (((h.y >> (8 * J + 6)) & 3u) << 4);
        sc1 = ((h.w >> (8 * J + 8)) & 0xFu) | (((h.y >> (8 * J + 14)) & 3u) << 4);
        m0 = ((h.w >> (8 * J + 4)) & 0xFu) | (((h.z >> (8 * J + 6)) & 3u) << 4);
        m1 = ((h.w >> (8 * J + 12)) & 0xFu) | (((h.z >> (8 * J + 14)) & 3u) << 4);
    }
    const float d = h2f(h.x & 0xFFFFu), dmin = h2f(h.x >> 16);
    const float ds0 = d * (float)sc0, dm0 = dmin * (float)m0, ds1 = d * (float)sc1, dm1 = dmin * (float)m1;
    const uint4 qa = blk[1 + 2 * P], qb = blk[2 + 2 * P];
    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        uint4 lo, hi;
        nib4_to_h2(w[2 * c] & 0x0F0F0F0Fu, ds0, dm0, lo.x, lo.y);
        nib4_to_h2(w[2 * c + 1] & 0x0F0F0F0Fu, ds0, dm0, lo.z, lo.w);
        nib4_to_h2((w[2 * c] >> 4) & 0x0F0F0F0Fu, ds1, dm1, hi.x, hi.y);
        nib4_to_h2((w[2 * c + 1] >> 4) & 0x0F0F0F0Fu, ds1, dm1, hi.z, hi.w);
        sts128(rowaddr + (((uint32_t)c ^ r7) << 4), lo);
        sts128(rowaddr + (((uint32_t)(c + 4) ^ r7) << 4), hi);
    }
}

// Any format: eight consecutive weights at a time through the exact scalar decode.
template <int FMT>
__device__ __forceinline__ void generic_kb_to_smem(const uint8_t* row, int kb, uint32_t rowaddr, uint32_t r7) {
#pragma unroll 2
    for (int c = 0; c < 8; ++c) {
        float w[8];
        decode8<FMT>(row, kb * 8 + c, w);
        uint4 o;
        o.x = pack_h2(w[0], w[1]); o.y = pack_h2(w[2], w[3]); o.z = pack_h2(w[4], w[5]); o.w = pack_h2(w[6], w[7]);
        sts128(rowaddr + (((uint32_t)c ^ r7) << 4), o);
    }
}

__device__ __forceinline__ bool gemm_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
    return wait_or_abort(bar, parity, abort_flag, status, code);
}

}  // namespace b200q

// Streaming decode GEMV with integer dot products, 1..4 activation rows (sm_100a).
//
// Same pipeline as gemv_stream.cu (persistent grid, one contiguous row range per
// CTA, producer warp + bulk-copy ring), different consumers. The bottleneck of a
// decode GEMV at 6.5 TB/s is instruction issue, so the inner loop is cut to the
// minimum: quants stay integers and are multiplied by 16-bit fixed-point
// activations with dp2a (two 16-bit x 8-bit products per lane and instruction).
//
//   * Activations are staged once per CTA: every group of 128 consecutive x values
//     gets its own power-of-two scale 2^e so that |x| * 2^e < 2^14, the values are
//     rounded to int16, and the group's 2^-e is kept as a float. The worst-case
//     relative error of a group's contribution is about sqrt(128) / 2^15 = 3.5e-4,
//     typically 7e-5 - an outlier only costs precision inside its own group.
//   * Each warp owns two weight rows of the 16-row stage, each lane one 128-element
//     group of both rows per step, so the activations of a group are loaded once
//     for two rows. Q4_K nibbles need three integer ops per eight weights
//     (two masks, one shift), Q6_K builds its 6-bit values with shifts and masks,
//     Q8_0 bytes feed dp2a directly.
//   * Sub-block scales are applied to the integer sums (Q4_K: in integers, four
//     sub-blocks per conversion; Q6_K and Q8_0: one int->float per sub-block /
//     block), the block scale and the group's 2^-e in FP32. Decode is exact:
//     everything up to the final FP32 accumulation is integer arithmetic.
//   * No cross-warp reduction: a row's partial sums live in the 32 lanes of one
//     warp and are combined with shuffles when the row's last slice is done.
//
// Takes the place of brotensor's linear_q4k_fp16_gemv_kernel
// (src/cuda/q4k.cu:159-224), linear_q6k_fp16_gemv_kernel (q6k.cu:117-176) and
// linear_q8_0_fp16_gemv_kernel (q8_0.cu:75-138), and of the per-row GEMV loop the
// batched ops fall back to for small B (q4k.cu:413-418).
#include "stream_common.cuh"
#include "dp_common.cuh"

namespace b200q {

// One segment (eight consecutive activations) of the staged image; called by whole warps.
// (Inlined on purpose: as a function of its own it cost every launch close to a microsecond.)
template <int FMT>
__device__ __forceinline__ void x_store_seg(
    const StreamParams& p, uint32_t sbase, int idx, float4 lo, float4 hi) {
    const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    const int segs = p.K >> 3, groups = p.K >> 7;
    const int m = idx / segs, seg = idx - m * segs;
    const int gg = seg >> 4, i = seg & 15;
    float amax = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(v[k]));
    // the 16 segments of a group are 16 consecutive lanes
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 8));
    // 2^e with amax * 2^e in [2^13, 2^14); e clamped so both 2^e and 2^-e are normal floats
    int e = 0;
    if (amax > 0.f && amax < 3.0e38f) e = 13 - (int)((__float_as_uint(amax) >> 23) & 0xFFu) + 127;
    e = max(-126, min(126, e));
    const float s = __uint_as_float((uint32_t)(e + 127) << 23);
    int q[8], sum = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        q[k] = max(-16383, min(16383, __float2int_rn(v[k] * s)));
        sum += q[k];
    }
    uint4 o;
    o.x = (uint32_t)(q[0] & 0xFFFF) | ((uint32_t)q[1] << 16);
    o.y = (uint32_t)(q[2] & 0xFFFF) | ((uint32_t)q[3] << 16);
    o.z = (uint32_t)(q[4] & 0xFFFF) | ((uint32_t)q[5] << 16);
    o.w = (uint32_t)(q[6] & 0xFFFF) | ((uint32_t)q[7] << 16);
    sts128(sbase + p.off_xhi + (uint32_t)((m * groups + gg) * kXGroupStride + (i << 4)), o);
    if (i == 0) sts32(sbase + p.off_xlo + (uint32_t)(m * groups + gg) * 4, (uint32_t)(127 - e) << 23);
    if constexpr (FMT == kQ4_K) {  // sums over 32 elements = 4 segments
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if ((i & 3) == 0) sts32(sbase + p.off_sxhi + (uint32_t)(m * (p.K >> 5) + (seg >> 2)) * 4, (uint32_t)sum);
    } else if constexpr (FMT == kQ6_K || FMT == kQ6_KP) {  // sums over 16 elements = 2 segments
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        if ((i & 1) == 0) sts32(sbase + p.off_sxhi + (uint32_t)(m * (p.K >> 4) + (seg >> 1)) * 4, (uint32_t)sum);
    }
}

// Stages the activations as int16 with one power-of-two scale per 128-element group. A thread's
// global loads go out four segments at a time before any of them is converted, so a long row
// (K = 14336: 3.5 segments per thread) costs one load latency instead of one per segment.
template <int FMT, bool kLean = false>
__device__ __forceinline__ void stage_x16(const StreamParams& p, uint32_t sbase, int tid, int nthreads) {
    const int total = (p.K >> 3) * p.M;  // K % 256 == 0, so a multiple of 32: whole warps are in or out
    if (kLean || total <= nthreads) {  // at most one segment per thread (K = 4096, one activation row)
        if (tid < total) {
            float v[8];
            x_load_seg(p.X, kLean ? B200Q_DT_F32 : p.x_dtype, p.K, tid, v);
            x_store_seg<FMT>(p, sbase, tid, make_float4(v[0], v[1], v[2], v[3]), make_float4(v[4], v[5], v[6], v[7]));
        }
        return;
    }
    // Four segments per thread and pass. The loads are unconditional (a segment past the end re-reads
    // the last one) and the element type is switched once around them, so that all four go out before
    // the first conversion: behind a condition each one waited for the one before it (K = 14336,
    // 3.5 segments per thread: 2.6 us of staging, one load latency per segment).
    const int segs = p.K >> 3;
    for (int base = tid; base < total; base += 4 * nthreads) {
        float v[4][8];
        if (p.x_dtype == B200Q_DT_F32) {
            float4 r[4][2];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int idx = min(base + u * nthreads, total - 1), m = idx / segs, seg = idx - m * segs;
                const float4* X = reinterpret_cast<const float4*>(static_cast<const float*>(p.X) + (size_t)m * p.K) + 2 * seg;
                r[u][0] = __ldg(X);
                r[u][1] = __ldg(X + 1);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                v[u][0] = r[u][0].x; v[u][1] = r[u][0].y; v[u][2] = r[u][0].z; v[u][3] = r[u][0].w;
                v[u][4] = r[u][1].x; v[u][5] = r[u][1].y; v[u][6] = r[u][1].z; v[u][7] = r[u][1].w;
            }
        } else {
            uint4 r[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int idx = min(base + u * nthreads, total - 1), m = idx / segs, seg = idx - m * segs;
                r[u] = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.X) + (size_t)m * p.K) + seg);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t w[4] = {r[u].x, r[u].y, r[u].z, r[u].w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (p.x_dtype == B200Q_DT_F16) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
                        v[u][2 * k] = f.x;
                        v[u][2 * k + 1] = f.y;
                    } else {  // BF16: the upper half of an FP32
                        v[u][2 * k] = __uint_as_float(w[k] << 16);
                        v[u][2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (base + u * nthreads < total)
                x_store_seg<FMT>(p, sbase, base + u * nthreads, make_float4(v[u][0], v[u][1], v[u][2], v[u][3]), make_float4(v[u][4], v[u][5], v[u][6], v[u][7]));
    }
}

// The same staging with brotensor's rms_norm_forward (src/cuda/rms_norm.cu:56-75: FP32 sum of squares,
// rsqrtf(sum / D + eps), times gamma) folded in, one activation row: every CTA computes the row's
// scale itself (K values from L2), so the normalised vector is never written out and the
// normalisation costs no launch. `red` is 32 floats of shared memory; called by `nthreads`
// threads that meet on named barrier 1.
template <int FMT>
__device__ __forceinline__ void stage_x16_norm(const StreamParams& p, uint32_t sbase, int tid, int nthreads, float* red) {
    const int total = p.K >> 3;  // a multiple of 32: whole warps are in or out
    float ss = 0.f;
    for (int idx = tid; idx < total; idx += nthreads) {
        float v[8];
        x_load_seg(p.X, p.x_dtype, p.K, idx, v);
#pragma unroll
        for (int k = 0; k < 8; ++k) ss = fmaf(v[k], v[k], ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    float sum = 0.f;
    for (int w = 0; w < (nthreads >> 5); ++w) sum += red[w];  // the same order in every thread
    const float rr = rsqrtf(sum / (float)p.K + p.norm_eps);
    for (int idx = tid; idx < total; idx += nthreads) {
        float v[8], w[8];
        x_load_seg(p.X, p.x_dtype, p.K, idx, v);
        x_load_seg(p.norm_gamma, p.x_dtype, p.K, idx, w);  // gamma is read like an activation row
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = v[k] * rr * w[k];
        x_store_seg<FMT>(p, sbase, idx, make_float4(v[0], v[1], v[2], v[3]), make_float4(v[4], v[5], v[6], v[7]));
    }
}

// Shared-memory addresses an item needs for the staged activations.
struct XAddr {
    uint32_t x16, xsc, sxi;  // region bases
    int groups, K;
};
__device__ __forceinline__ uint32_t x_group(const XAddr& xa, int m, int gg) {
    return xa.x16 + (uint32_t)((m * xa.groups + gg) * kXGroupStride);
}
template <int I>
__device__ __forceinline__ uint4 x_seg(uint32_t xg) { return lds128i<16 * I>(xg); }

// ---- one item = one 128-element group of two weight rows ---------------------------
// rowA/rowB: shared addresses of this stage's bytes of the two rows; gi: group index
// inside the stage; gg: group index along the whole row; acc[r][m]: FP32 partial sums.
// Loads are written in the order they should issue (the asm statements keep it): all
// weight loads of the item first, activations one step ahead of their use.

template <int C2>
__device__ __forceinline__ void q4k_load_x(uint32_t xg, uint4 (&x)[8]) {
    x[0] = x_seg<8 * C2 + 0>(xg); x[1] = x_seg<8 * C2 + 1>(xg); x[2] = x_seg<8 * C2 + 2>(xg); x[3] = x_seg<8 * C2 + 3>(xg);
    x[4] = x_seg<8 * C2 + 4>(xg); x[5] = x_seg<8 * C2 + 5>(xg); x[6] = x_seg<8 * C2 + 6>(xg); x[7] = x_seg<8 * C2 + 7>(xg);
}

template <int MT>
__device__ __forceinline__ void item_q4k(uint32_t rowA, uint32_t rowB, int gi, int gg, const XAddr& xa,
                                         float (&acc)[2][MT]) {
    const int b = gi >> 1, hb = gi & 1;
    const uint32_t prA = rowA + (uint32_t)b * 144u, prB = rowB + (uint32_t)b * 144u;
    const uint32_t qaA = prA + 64u * hb, qaB = prB + 64u * hb;
    const uint4 hA = lds128i<0>(prA), hB = lds128i<0>(prB);
    uint4 q[2][2][2];  // [c2][row][half]
    q[0][0][0] = lds128i<16>(qaA); q[0][0][1] = lds128i<32>(qaA);
    q[0][1][0] = lds128i<16>(qaB); q[0][1][1] = lds128i<32>(qaB);
    // activations: x0 serves chunk 0, x1 chunk 1 of activation row m; the loads of the
    // next step are written before the math of the current one
    uint4 x0[8], x1[8];
    const uint32_t xg0 = x_group(xa, 0, gg);
    q4k_load_x<0>(xg0, x0);
    q[1][0][0] = lds128i<48>(qaA); q[1][0][1] = lds128i<64>(qaA);
    q[1][1][0] = lds128i<48>(qaB); q[1][1][1] = lds128i<64>(qaB);
    q4k_load_x<1>(xg0, x1);

    // the four 6-bit scales / mins of sub-blocks 4*hb .. 4*hb+3, one per byte
    uint32_t scw[2], mw[2];
    float d[2], dm[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint4 h = r ? hB : hA;
        const uint32_t sclo = h.y & 0x3f3f3f3fu, schi = (h.w & 0x0f0f0f0fu) | ((h.y >> 2) & 0x30303030u);
        const uint32_t mlo = h.z & 0x3f3f3f3fu, mhi = ((h.w >> 4) & 0x0f0f0f0fu) | ((h.z >> 2) & 0x30303030u);
        scw[r] = hb ? schi : sclo;
        mw[r] = hb ? mhi : mlo;
        d[r] = h2f(h.x & 0xFFFFu);
        dm[r] = h2f(h.x >> 16);
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        int isum[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            int cl, ch;
            q4k_dot(q[0][r][0], q[0][r][1], x0, cl, ch);
            // |sc * c| <= 63 * 32*15*16383 = 4.95e8 and four of them fit an int32
            isum[r] = (int)(scw[r] & 0xFFu) * cl + (int)((scw[r] >> 8) & 0xFFu) * ch;
        }
        if (m + 1 < MT) q4k_load_x<0>(x_group(xa, m + 1, gg), x0);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            int cl, ch;
            q4k_dot(q[1][r][0], q[1][r][1], x1, cl, ch);
            isum[r] += (int)((scw[r] >> 16) & 0xFFu) * cl + (int)(scw[r] >> 24) * ch;
        }
        if (m + 1 < MT) q4k_load_x<1>(x_group(xa, m + 1, gg), x1);
        const uint4 sv = lds128i<0>(xa.sxi + (uint32_t)(m * (xa.K >> 5) + gg * 4) * 4u);
        const float xs = __uint_as_float(lds32i<0>(xa.xsc + (uint32_t)(m * xa.groups + gg) * 4u));
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int imin = (int)(mw[r] & 0xFFu) * (int)sv.x + (int)((mw[r] >> 8) & 0xFFu) * (int)sv.y +
                             (int)((mw[r] >> 16) & 0xFFu) * (int)sv.z + (int)(mw[r] >> 24) * (int)sv.w;
            acc[r][m] = fmaf(xs, d[r] * (float)isum[r] - dm[r] * (float)imin, acc[r][m]);
        }
    }
}

// The same item for two to four activation rows, ordered for registers instead of load distance:
// with both chunks' quants and two activation chunks live (item_q4k) the kernel spills under the
// 96-register cap of an 18-warp CTA; here one chunk of quants (16 registers) and one chunk of one
// row's activations (32) are live at a time.
template <int MT>
__device__ __forceinline__ void item_q4k_rows(uint32_t rowA, uint32_t rowB, int gi, int gg, const XAddr& xa,
                                              float (&acc)[2][MT]) {
    const int b = gi >> 1, hb = gi & 1;
    const uint32_t prA = rowA + (uint32_t)b * 144u, prB = rowB + (uint32_t)b * 144u;
    const uint32_t qaA = prA + 64u * hb, qaB = prB + 64u * hb;
    const uint4 hA = lds128i<0>(prA), hB = lds128i<0>(prB);
    uint32_t scw[2], mw[2];
    float d[2], dm[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint4 h = r ? hB : hA;
        const uint32_t sclo = h.y & 0x3f3f3f3fu, schi = (h.w & 0x0f0f0f0fu) | ((h.y >> 2) & 0x30303030u);
        const uint32_t mlo = h.z & 0x3f3f3f3fu, mhi = ((h.w >> 4) & 0x0f0f0f0fu) | ((h.z >> 2) & 0x30303030u);
        scw[r] = hb ? schi : sclo;
        mw[r] = hb ? mhi : mlo;
        d[r] = h2f(h.x & 0xFFFFu);
        dm[r] = h2f(h.x >> 16);
    }
    int isum[2][MT];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) isum[r][m] = 0;
    {
        const uint4 a0 = lds128i<16>(qaA), a1 = lds128i<32>(qaA), b0 = lds128i<16>(qaB), b1 = lds128i<32>(qaB);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            uint4 x[8];
            q4k_load_x<0>(x_group(xa, m, gg), x);
            int cl, ch;
            q4k_dot(a0, a1, x, cl, ch);
            isum[0][m] = (int)(scw[0] & 0xFFu) * cl + (int)((scw[0] >> 8) & 0xFFu) * ch;
            q4k_dot(b0, b1, x, cl, ch);
            isum[1][m] = (int)(scw[1] & 0xFFu) * cl + (int)((scw[1] >> 8) & 0xFFu) * ch;
        }
    }
    {
        const uint4 a0 = lds128i<48>(qaA), a1 = lds128i<64>(qaA), b0 = lds128i<48>(qaB), b1 = lds128i<64>(qaB);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            uint4 x[8];
            q4k_load_x<1>(x_group(xa, m, gg), x);
            int cl, ch;
            q4k_dot(a0, a1, x, cl, ch);
            isum[0][m] += (int)((scw[0] >> 16) & 0xFFu) * cl + (int)(scw[0] >> 24) * ch;
            q4k_dot(b0, b1, x, cl, ch);
            isum[1][m] += (int)((scw[1] >> 16) & 0xFFu) * cl + (int)(scw[1] >> 24) * ch;
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const uint4 sv = lds128i<0>(xa.sxi + (uint32_t)(m * (xa.K >> 5) + gg * 4) * 4u);
        const float xs = __uint_as_float(lds32i<0>(xa.xsc + (uint32_t)(m * xa.groups + gg) * 4u));
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int imin = (int)(mw[r] & 0xFFu) * (int)sv.x + (int)((mw[r] >> 8) & 0xFFu) * (int)sv.y +
                             (int)((mw[r] >> 16) & 0xFFu) * (int)sv.z + (int)(mw[r] >> 24) * (int)sv.w;
            acc[r][m] = fmaf(xs, d[r] * (float)isum[r][m] - dm[r] * (float)imin, acc[r][m]);
        }
    }
}

template <int J>
__device__ __forceinline__ void q8_block_words(uint32_t base, uint32_t (&w)[9]) {
    // block J of the group starts at 34*J: 4-byte aligned for even J, 2 (mod 4) for odd J
    constexpr int O = (J & 1) ? 34 * J - 2 : 34 * J;
    w[0] = lds32i<O>(base);      w[1] = lds32i<O + 4>(base);  w[2] = lds32i<O + 8>(base);
    w[3] = lds32i<O + 12>(base); w[4] = lds32i<O + 16>(base); w[5] = lds32i<O + 20>(base);
    w[6] = lds32i<O + 24>(base); w[7] = lds32i<O + 28>(base); w[8] = lds32i<O + 32>(base);
}

template <int MT, int J>
__device__ __forceinline__ void q8_block(const uint32_t (&pr)[2], int gg, const XAddr& xa, float (&acc)[2][MT]) {
    uint32_t w[2][9];
    q8_block_words<J>(pr[0], w[0]);
    q8_block_words<J>(pr[1], w[1]);
    uint4 xv[MT][4];
    float xs[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const uint32_t xg = x_group(xa, m, gg);
        xv[m][0] = x_seg<4 * J>(xg); xv[m][1] = x_seg<4 * J + 1>(xg);
        xv[m][2] = x_seg<4 * J + 2>(xg); xv[m][3] = x_seg<4 * J + 3>(xg);
        xs[m] = __uint_as_float(lds32i<0>(xa.xsc + (uint32_t)(m * xa.groups + gg) * 4u));
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        uint32_t qs[8];
        float d;
        if (J & 1) {
            d = h2f(w[r][0] >> 16);
#pragma unroll
            for (int k = 0; k < 8; ++k) qs[k] = w[r][k + 1];
        } else {
            d = h2f(w[r][0] & 0xFFFFu);
#pragma unroll
            for (int k = 0; k < 8; ++k) qs[k] = __byte_perm(w[r][k], w[r][k + 1], 0x5432);
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            int c0 = 0, c1 = 0;
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                c0 = dp2a_lo_ss(xv[m][s].x, qs[2 * s], c0);
                c0 = dp2a_hi_ss(xv[m][s].y, qs[2 * s], c0);
                c1 = dp2a_lo_ss(xv[m][s].z, qs[2 * s + 1], c1);
                c1 = dp2a_hi_ss(xv[m][s].w, qs[2 * s + 1], c1);
            }
            acc[r][m] = fmaf(d * xs[m], (float)(c0 + c1), acc[r][m]);
        }
    }
}

template <int MT>
__device__ __forceinline__ void item_q8_0(uint32_t rowA, uint32_t rowB, int gi, int gg, const XAddr& xa,
                                          float (&acc)[2][MT]) {
    const uint32_t pr[2] = {rowA + (uint32_t)gi * 136u, rowB + (uint32_t)gi * 136u};  // four 34-byte blocks
    q8_block<MT, 0>(pr, gg, xa, acc);
    q8_block<MT, 1>(pr, gg, xa, acc);
    q8_block<MT, 2>(pr, gg, xa, acc);
    q8_block<MT, 3>(pr, gg, xa, acc);
}

// int8 scale byte `idx` of a word whose bytes were xor-ed with 0x80 -> exact float
__device__ __forceinline__ float biased_s8_to_f32(uint32_t u, int idx) {
    return __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7440 | idx)) - 8388736.0f;  // 2^23 + 128
}

template <int N, int K0 = 0>
__device__ __forceinline__ void load_words(uint32_t a, uint32_t* out) {
    if constexpr (K0 < N) {
        out[K0] = lds32i<4 * K0>(a);
        load_words<N, K0 + 1>(a, out);
    }
}

// ---- Q6_K in units of half a group --------------------------------------------------------
// The 64 elements {32 Q + 16 H + i : Q = 0..3, i = 0..15} of a 128-element group use ql words
// 4H..4H+3 and 4H+8..4H+11 and qh words 4H..4H+3 of the group's bytes - half of its loads - so
// a lane can take (group, H) as its unit of work: 32 lanes then cover 16 groups (one 2048-element
// chunk), slices can be half as long and two pipelines fit beside a long activation vector.
template <int MT, int Q>
__device__ __forceinline__ void q6_sub_h(const uint32_t (&ql)[2][8], const uint32_t (&qh)[2][4], const uint32_t (&su)[2][2],
                                         int H, int gg, const XAddr& xa, float (&accg)[2][MT]) {
    const int SI = 2 * Q + H;  // scale byte and 16-element sum index inside the group
    uint4 x0[MT], x1[MT];
    int sx[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const uint32_t xg = x_group(xa, m, gg) + (uint32_t)(32 * H);
        x0[m] = lds128i<64 * Q>(xg);
        x1[m] = lds128i<64 * Q + 16>(xg);
        sx[m] = (int)lds32i<8 * Q>(xa.sxi + (uint32_t)((m * (xa.K >> 4) + gg * 8 + H) * 4));
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        uint32_t v[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const uint32_t a = ql[r][4 * (Q & 1) + w], hb = qh[r][w];
            const uint32_t nib = (Q < 2 ? a : (a >> 4)) & 0x0F0F0F0Fu;
            const uint32_t h2 = (Q == 0 ? hb << 4 : Q == 1 ? hb << 2 : Q == 2 ? hb : hb >> 2) & 0x30303030u;
            v[w] = nib | h2;
        }
        const float scf = biased_s8_to_f32(su[r][Q >> 1], 2 * (Q & 1) + H);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            int c0 = 0, c1 = 0;
            c0 = dp2a_lo_su(x0[m].x, v[0], c0);
            c0 = dp2a_hi_su(x0[m].y, v[0], c0);
            c1 = dp2a_lo_su(x0[m].z, v[1], c1);
            c1 = dp2a_hi_su(x0[m].w, v[1], c1);
            c0 = dp2a_lo_su(x1[m].x, v[2], c0);
            c0 = dp2a_hi_su(x1[m].y, v[2], c0);
            c1 = dp2a_lo_su(x1[m].z, v[3], c1);
            c1 = dp2a_hi_su(x1[m].w, v[3], c1);
            accg[r][m] = fmaf(scf, (float)(c0 + c1 - 32 * sx[m]), accg[r][m]);
        }
    }
}

template <int MT>
__device__ __forceinline__ void item_q6k_half(uint32_t rowA, uint32_t rowB, int gi, int H, int gg, const XAddr& xa,
                                              float (&acc)[2][MT]) {
    const int bi = gi >> 1, G = gi & 1;
    const uint32_t sh = (uint32_t)(bi & 1) * 16u;  // odd blocks start at 2 (mod 4): aligned words + funnel shift
    uint32_t ql[2][8], qh[2][4], su[2][2];
    float d[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint32_t L = (r ? rowB : rowA) + (uint32_t)(bi * 210 - (bi & 1) * 2);
        const uint32_t La = L + 64u * G + 16u * H, Lh = L + 128u + 32u * G + 16u * H, Ls = L + 192u + 8u * G;
        uint32_t ra[5], rb[5], rh[5], rs[3];
        load_words<5>(La, ra);
        load_words<5>(La + 32u, rb);
        load_words<5>(Lh, rh);
        load_words<3>(Ls, rs);
        const uint32_t rd = lds32i<208>(L);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            ql[r][k] = __funnelshift_r(ra[k], ra[k + 1], sh);
            ql[r][4 + k] = __funnelshift_r(rb[k], rb[k + 1], sh);
            qh[r][k] = __funnelshift_r(rh[k], rh[k + 1], sh);
        }
        su[r][0] = __funnelshift_r(rs[0], rs[1], sh) ^ 0x80808080u;
        su[r][1] = __funnelshift_r(rs[1], rs[2], sh) ^ 0x80808080u;
        d[r] = h2f((rd >> sh) & 0xFFFFu);
    }
    float accg[2][MT];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) accg[r][m] = 0.f;
    q6_sub_h<MT, 0>(ql, qh, su, H, gg, xa, accg);
    q6_sub_h<MT, 1>(ql, qh, su, H, gg, xa, accg);
    q6_sub_h<MT, 2>(ql, qh, su, H, gg, xa, accg);
    q6_sub_h<MT, 3>(ql, qh, su, H, gg, xa, accg);
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const float xs = __uint_as_float(lds32i<0>(xa.xsc + (uint32_t)(m * xa.groups + gg) * 4u));
#pragma unroll
        for (int r = 0; r < 2; ++r) acc[r][m] = fmaf(d[r] * xs, accg[r][m], acc[r][m]);
    }
}

// The same half-group item on the layout regrouped by field in runs of eight blocks (b200q_repack):
// every field sits on a 16-byte boundary, so the item's bytes come in three 16-byte loads, one
// 8-byte load and one word per row instead of nineteen words and fourteen funnel shifts.
template <int MT>
__device__ __forceinline__ void item_q6kp_half(uint32_t rowA, uint32_t rowB, int gi, int H, int gg, const XAddr& xa,
                                               float (&acc)[2][MT]) {
    const int run = gi >> 4, bi = (gi >> 1) & 7, G = gi & 1;  // sixteen groups per run; block slot; half of the block
    uint32_t ql[2][8], qh[2][4], su[2][2];
    float d[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint32_t R = (r ? rowB : rowA) + (uint32_t)(run * kQ6RunBytes);
        // The two 16-byte pieces sit 32 bytes apart and groups 64 bytes apart, so with every lane
        // reading its first piece first a warp would touch four of the eight 16-byte bank groups;
        // lanes of odd blocks read the second piece first and swap afterwards.
        const uint32_t sw = (uint32_t)(bi & 1);
        const uint32_t pa = R + (uint32_t)(bi * 128 + 64 * G + 16 * H);
        const uint4 t0 = lds128i<0>(pa + 32u * sw), t1 = lds128i<0>(pa + 32u * (sw ^ 1u));
        const uint4 a = sw ? t1 : t0, b = sw ? t0 : t1;
        const uint4 h = lds128i<1024>(R + (uint32_t)(bi * 64 + 32 * G + 16 * H));
        const uint2 sc = lds64(R + (uint32_t)(1536 + bi * 16 + 8 * G));
        const uint32_t dw = lds32i<1664>(R + (uint32_t)((bi >> 1) * 4));
        ql[r][0] = a.x; ql[r][1] = a.y; ql[r][2] = a.z; ql[r][3] = a.w;
        ql[r][4] = b.x; ql[r][5] = b.y; ql[r][6] = b.z; ql[r][7] = b.w;
        qh[r][0] = h.x; qh[r][1] = h.y; qh[r][2] = h.z; qh[r][3] = h.w;
        su[r][0] = sc.x ^ 0x80808080u;
        su[r][1] = sc.y ^ 0x80808080u;
        d[r] = h2f((dw >> ((bi & 1) * 16)) & 0xFFFFu);
    }
    float accg[2][MT];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) accg[r][m] = 0.f;
    q6_sub_h<MT, 0>(ql, qh, su, H, gg, xa, accg);
    q6_sub_h<MT, 1>(ql, qh, su, H, gg, xa, accg);
    q6_sub_h<MT, 2>(ql, qh, su, H, gg, xa, accg);
    q6_sub_h<MT, 3>(ql, qh, su, H, gg, xa, accg);
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const float xs = __uint_as_float(lds32i<0>(xa.xsc + (uint32_t)(m * xa.groups + gg) * 4u));
#pragma unroll
        for (int r = 0; r < 2; ++r) acc[r][m] = fmaf(d[r] * xs, accg[r][m], acc[r][m]);
    }
}

// Order of the LM head's candidates: larger value first, among equal values the lower index
// (brotensor's greedy rule, include/brotensor/ops/sampling.h:27-28: "ties keep the lowest index").
__device__ __forceinline__ bool cand_before(float va, int ia, float vb, int ib) { return va > vb || (va == vb && ia < ib); }

// The k best of the candidates the CTA's threads hold (C each; unused ones are (-inf, INT_MAX)), in
// the candidates' order, left in scr[64 .. 64 + k) (values) and scr[64 + kMaxTopK ..) (rows): k
// passes, each taking the best candidate that comes after the previous pick. Called by all `nthreads`
// threads (named barrier 1); scr[32 .. 64 + 2 * kMaxTopK) is scratch.
template <int C>
__device__ __forceinline__ void block_topk(const float (&v)[C], const int (&ix)[C], int k, uint32_t* scr, int tid, int nthreads) {
    const int nwarps = nthreads >> 5;
    float pv = __int_as_float(0x7f800000);  // +inf
    int pi = -1;
    for (int r = 0; r < k; ++r) {
        float bv = __int_as_float(0xff800000);  // -inf
        int bi = 0x7fffffff;
#pragma unroll
        for (int u = 0; u < C; ++u)
            if (cand_before(pv, pi, v[u], ix[u]) && cand_before(v[u], ix[u], bv, bi)) { bv = v[u]; bi = ix[u]; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (cand_before(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if ((tid & 31) == 0) {
            scr[32 + 2 * (tid >> 5)] = __float_as_uint(bv);
            scr[33 + 2 * (tid >> 5)] = (uint32_t)bi;
        }
        asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
        bv = __uint_as_float(scr[32]);
        bi = (int)scr[33];
        for (int w = 1; w < nwarps; ++w) {  // the same order in every thread
            const float ov = __uint_as_float(scr[32 + 2 * w]);
            const int oi = (int)scr[33 + 2 * w];
            if (cand_before(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        pv = bv;
        pi = bi;
        if (tid == 0) {  // fewer than k candidates leave (-inf, INT_MAX)
            scr[64 + r] = __float_as_uint(bv);
            scr[64 + kMaxTopK + r] = (uint32_t)bi;
        }
        asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    }
}

// Sharded epilogue, run by all `nthreads` consumer threads of a CTA (thread ids 0 .. nthreads-1) after
// they have stored the CTA's rows [row_begin, row_end) into this rank's result vector. `scr` is
// shared memory that nothing else uses any more (1 KB; 8 * 2048 * k bytes more in the candidate form
// with k > 1).
//
// Nothing on the exchange path is a fence, a flag or a counter: every word that crosses the links
// validates itself. An aligned 8-byte store is indivisible, so a word that carries its payload in
// one half and the call's number in the other is either the old word or the new one, and the
// receiver simply polls it until the number is this call's (bounded; a word that never comes sets
// the timeout status). A rank can run at most one call ahead of a peer - it needs the peer's words
// of the call before - so two buffers, used alternately, are enough.
//
// Full-logits form (sh_topk == 0): the CTA sends its rows to every peer as (value, call number) words
// - coalesced, 256 bytes per warp and peer - and then receives ITS SLICE of the whole vector: it
// polls the words the peers have sent for rows [cta, cta + 1) * ceil(total / grid) and writes the
// values into this rank's result vector. When every CTA has done so the kernel - and with it the
// vector - is complete; the CTA that finishes last (a gpu-scope counter, off the data path) only
// advances the call numbers.
//
// Candidate form (sh_topk = k in 1..8): every CTA of every rank reduces its rows to k candidates and
// stores them - value, row (20 bits) and a 12-bit tag of the candidate-form call count per word - into
// EVERY rank's table, which has 256 slots per rank: a CTA also fills the slots of the CTA numbers its
// grid does not have ((-inf, no row)), so a receiver needs to know nobody's grid. CTA 0 of each
// rank polls the 8 x 256 x k words, takes the k best in the candidates' order and leaves them in
// sh_top_val / sh_top_idx; no CTA waits for another one of its own rank, and there is no atomic.
__device__ __forceinline__ void shard_publish(const StreamParams& p, int row_begin, int row_end, unsigned int sh_epoch,
                                              unsigned int sh_buf, int tid, int nthreads, uint32_t* scr, float top_v, int top_i, unsigned int cc) {
    // Every consumer warp gets here (aborted ones too).
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    const int k = p.sh_topk;
    const unsigned int epoch = sh_epoch + 1u;
    const uint64_t limit = p.wait_limit_us ? (uint64_t)p.wait_limit_us * 1000ull : kWaitLimitNs;
    if (k == 0) {
        if (p.sh_world > 1) {
            // transfer words of rank q: behind its two result vectors, [2][sh_total] x 8 bytes
            const size_t at = (size_t)sh_buf * p.sh_total;
            const float* own = p.sh_out[p.sh_rank] + at + (size_t)(p.sh_row_offset + row_begin);
            for (int i = tid; i < row_end - row_begin; i += nthreads) {
                const unsigned long long w = (unsigned long long)__float_as_uint(__ldcg(own + i)) | ((unsigned long long)epoch << 32);
                for (int q = 0; q < p.sh_world; ++q)
                    if (q != p.sh_rank) {
                        unsigned long long* dst = reinterpret_cast<unsigned long long*>(p.sh_out[q] + 2 * (size_t)p.sh_total) + at + (size_t)(p.sh_row_offset + row_begin + i);
                        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(w) : "memory");
                    }
            }
            // receive this CTA's slice (rows of this rank's own shard are in place already)
            const int slice = (p.sh_total + (int)gridDim.x - 1) / (int)gridDim.x;
            const int r1 = min(p.sh_total, ((int)blockIdx.x + 1) * slice);
            const unsigned long long* src = reinterpret_cast<const unsigned long long*>(p.sh_out[p.sh_rank] + 2 * (size_t)p.sh_total) + at;
            float* dst = p.sh_out[p.sh_rank] + at;
            const uint64_t t0 = global_timer_ns();
            for (int r = (int)blockIdx.x * slice + tid; r < r1; r += nthreads) {
                if (r >= p.sh_row_offset && r < p.sh_row_offset + p.N) continue;
                for (;;) {
                    unsigned long long w;
                    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(src + r) : "memory");
                    if ((unsigned int)(w >> 32) == epoch) {
                        dst[r] = __uint_as_float((uint32_t)w);
                        break;
                    }
                    if (global_timer_ns() - t0 > limit) {  // a peer's rows never came
                        if (p.status) atomicCAS(p.status, 0, kDevTimeoutPeer);
                        break;
                    }
                }
            }
            asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
        }
        if (tid == 0) {
            unsigned int done;
            asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(done) : "l"(p.sh_state) : "memory");
            if (done == gridDim.x - 1) {
                p.sh_state[0] = 0;
                *(volatile unsigned int*)&p.sh_state[1] = epoch;
            }
        }
        return;
    }

    // ---- candidate form
    TRACE_STAMP(tid == 0, 9);
    const unsigned int tag = cc & 0xFFFu, par = cc & 1u;
    if (k == 1) {
        // the threads kept the best of the rows they stored: reduce over the CTA
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, top_v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, top_i, o);
            if (cand_before(ov, oi, top_v, top_i)) { top_v = ov; top_i = oi; }
        }
        if ((tid & 31) == 0) {
            scr[32 + 2 * (tid >> 5)] = __float_as_uint(top_v);
            scr[33 + 2 * (tid >> 5)] = (uint32_t)top_i;
        }
        asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
        if (tid < 32) {
            const int nwarps = nthreads >> 5;
            top_v = tid < nwarps ? __uint_as_float(scr[32 + 2 * tid]) : __int_as_float(0xff800000);
            top_i = tid < nwarps ? (int)scr[33 + 2 * tid] : 0x7fffffff;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, top_v, o);
                const int oi = __shfl_xor_sync(0xffffffffu, top_i, o);
                if (cand_before(ov, oi, top_v, top_i)) { top_v = ov; top_i = oi; }
            }
            if (tid == 0) {
                scr[64] = __float_as_uint(top_v);
                scr[64 + kMaxTopK] = (uint32_t)top_i;
            }
        }
        asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    } else {
        // the k best of this CTA's rows, from its piece of the result vector (at most four per thread in registers)
        const float* own = p.sh_out[p.sh_rank] + (size_t)sh_buf * p.sh_total + p.sh_row_offset + row_begin;
        float v[4];
        int ix[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = tid + u * nthreads;
            v[u] = i < row_end - row_begin ? __ldcg(own + i) : __int_as_float(0xff800000);
            ix[u] = i < row_end - row_begin ? p.sh_row_offset + row_begin + i : 0x7fffffff;
        }
        block_topk<4>(v, ix, k, scr, tid, nthreads);
    }
    // ---- send: candidate j of CTA slot c for rank q at [par][rank][c][j]; this CTA's own slot and the
    // slots of the CTA numbers its grid does not have
    for (int t = tid; t < p.sh_world * kMaxTopK; t += nthreads) {
        const int q = t / kMaxTopK, j = t % kMaxTopK;  // every slot is rewritten in every call, used or not
        unsigned long long* tab = reinterpret_cast<unsigned long long*>(p.sh_cand[q]) + ((size_t)par * kMaxShardRanks + p.sh_rank) * kShardSlots * kMaxTopK;
        const unsigned long long none = 0xff800000ull | ((unsigned long long)(0xFFFFFu | (tag << 20)) << 32);
        const uint32_t row = j < k ? scr[64 + kMaxTopK + j] : 0xFFFFFu;
        const unsigned long long w = j < k ? (unsigned long long)scr[64 + j] | ((unsigned long long)((row >= 0xFFFFFu ? 0xFFFFFu : row) | (tag << 20)) << 32) : none;
        for (int c = (int)blockIdx.x; c < kShardSlots; c += (int)gridDim.x) {
            unsigned long long* dst = tab + (size_t)c * kMaxTopK + j;
            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(c == (int)blockIdx.x ? w : none) : "memory");
        }
    }
    TRACE_STAMP(tid == 0, 10);
    if (blockIdx.x != 0) return;
    // ---- CTA 0 receives: all ranks' slots, candidates j < k
    const unsigned long long* tab = reinterpret_cast<const unsigned long long*>(p.sh_cand[p.sh_rank]) + (size_t)par * kMaxShardRanks * kShardSlots * kMaxTopK;
    const int n_words = p.sh_world * kShardSlots * k;
    const uint64_t t0 = global_timer_ns();
    bool ok = true;
    float bv = __int_as_float(0xff800000);
    int bi = 0x7fffffff;
    uint2* const pool = reinterpret_cast<uint2*>(scr + 256);  // k > 1: every received candidate, for the k passes below
    for (int t = tid; t < n_words; t += nthreads) {
        const int q = t / (kShardSlots * k), rem = t - q * kShardSlots * k, c = rem / k, j = rem - c * k;
        const unsigned long long* src = tab + ((size_t)q * kShardSlots + c) * kMaxTopK + j;
        float v = __int_as_float(0xff800000);
        int row = 0x7fffffff;
        for (;;) {
            unsigned long long w;
            asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(src) : "memory");
            if ((((unsigned int)(w >> 52)) & 0xFFFu) == tag) {
                v = __uint_as_float((uint32_t)w);
                const unsigned int rw = (unsigned int)(w >> 32) & 0xFFFFFu;
                row = rw == 0xFFFFFu ? 0x7fffffff : (int)rw;
                break;
            }
            if (global_timer_ns() - t0 > limit) {  // a peer's candidates never came
                if (p.status) atomicCAS(p.status, 0, kDevTimeoutPeer);
                ok = false;
                break;
            }
        }
        if (k == 1) {
            if (cand_before(v, row, bv, bi)) { bv = v; bi = row; }
        } else {
            pool[t] = make_uint2(__float_as_uint(v), (uint32_t)row);
        }
    }
    TRACE_STAMP(tid == 0, 11);
    scr[1] = 1u;
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    TRACE_STAMP(tid == 0, 12);
    if (!ok) scr[1] = 0u;
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    ok = scr[1] != 0u;
    const int nwarps = nthreads >> 5;
    float pv = __int_as_float(0x7f800000);
    int pi = -1;
    for (int r = 0; r < k; ++r) {
        if (k > 1) {  // the best pooled candidate after the previous pick
            bv = __int_as_float(0xff800000);
            bi = 0x7fffffff;
            for (int t = tid; t < n_words; t += nthreads) {
                const uint2 e = pool[t];
                const float v = __uint_as_float(e.x);
                const int row = (int)e.y;
                if (cand_before(pv, pi, v, row) && cand_before(v, row, bv, bi)) { bv = v; bi = row; }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (cand_before(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if ((tid & 31) == 0) {
            scr[32 + 2 * (tid >> 5)] = __float_as_uint(bv);
            scr[33 + 2 * (tid >> 5)] = (uint32_t)bi;
        }
        asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
        bv = __uint_as_float(scr[32]);
        bi = (int)scr[33];
        for (int w = 1; w < nwarps; ++w) {  // the same order in every thread
            const float ov = __uint_as_float(scr[32 + 2 * w]);
            const int oi = (int)scr[33 + 2 * w];
            if (cand_before(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        pv = bv;
        pi = bi;
        if (tid == 0 && ok) {
            p.sh_top_val[r] = bv;
            p.sh_top_idx[r] = bi;
        }
        asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    }
    if (tid == 0) {
        *(volatile unsigned int*)&p.sh_state[2] = cc;
        *(volatile unsigned int*)&p.sh_state[1] = epoch;
    }
    TRACE_STAMP(tid == 0, 13);
}

// NG independent pipelines inside one CTA: pipeline g has eight consumer warps, its own
// producer warp, its own ring of p.n_stages stages and its own barriers, and works on
// the row tiles t with t % NG == g. The pipelines share only the staged activations,
// so twice as many warps hide each other's latencies without any coupling between
// their barrier phases.
// Where the tile that starts at virtual row `vrow` lives: which matrix, which of its rows.
struct TileRef {
    const uint8_t* W;
    void* Y;
    const void* bias;
    int N;     // rows of that matrix (leading dimension of its Y)
    int row0;  // first row of the tile inside that matrix
};
// Bits of the kernel's EXT template argument (see gemv_dp_kernel).
constexpr int kExtSeg = 1, kExtShard = 2, kExtNorm = 4, kExtSwiglu = 8;
// Not a form but a promise about the launch that lets the compiler drop code: FP32 activations and
// results, no bias, one slice per tile with one barrier per consumer warp, at most one staging
// segment per thread. The commonest decode call (hidden size 4096, one token) qualifies.
constexpr int kExtLean = 32;

template <int EXT>
__device__ __forceinline__ TileRef tile_ref(const StreamParams& p, int vrow) {
    if (!(EXT & kExtSeg) || p.n_seg <= 1) return {p.W, p.Y, p.bias, p.N, vrow};
    int s = 0;
#pragma unroll
    for (int i = 1; i < kMaxSegments; ++i)
        if (i < p.n_seg && vrow >= kTileRows * p.seg_tile0[i]) s = i;
    return {p.seg_W[s], p.seg_Y[s], p.seg_bias[s], p.seg_rows[s], vrow - kTileRows * p.seg_tile0[s]};
}

// RP = row pairs per consumer warp and tile: a tile has 16 * RP rows. Two pairs per warp double
// the bytes a tile moves per barrier round trip (what the per-tile overheads are paid on) and
// give every lane two independent chains of work.
// EXT is a mask of what a launch does beyond the plain GEMV: several matrices per launch, the
// row-sharded epilogue, RMSNorm folded into the staging, a gate / up pair with a SwiGLU epilogue.
// Each used combination is its own instantiation, so that no kernel carries code it does not run:
// a chain that alternates between kernels pays for every kernel's size at each switch (with the
// two fused forms compiled into the plain GEMV the seven-launch layer set took 49.2 instead of
// 44.0 us; with everything in one extended kernel the four-launch set took 40.9 instead of 35.6 us).
template <int FMT, int MT, int NG, int RP, int EXT = 0>
__global__ void __launch_bounds__((kConsumerWarps + 1) * NG * 32, 1) gemv_dp_kernel(const __grid_constant__ StreamParams p) {
    constexpr int TR = kTileRows * RP;
    // Q4_K and Q8_0 always run with one full barrier per consumer warp; only Q6_K chooses at run time.
    constexpr bool kLean = (EXT & kExtLean) != 0;
    constexpr bool kSplitAlways = (FMT != kQ6_K && FMT != kQ6_KP) || kLean;
    const bool split_full = kSplitAlways || p.split_full != 0;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 127u) & ~127u;  // shared-space address
    // With p.split_full, one full barrier per consumer warp and stage: a warp's rows complete on
    // their own barrier, so it starts on them as soon as they have landed instead of when the whole
    // tile has. That shortens what a launch cannot overlap - the wait for the first tile and the work
    // after the last. Otherwise one barrier per stage (long Q6_K streams, where the split gains nothing).
    __shared__ uint64_t bar_full[NG][kMaxStages][kConsumerWarps];
    __shared__ uint64_t bar_empty[NG][kMaxStages];
    __shared__ int abort_flag;
    __shared__ float norm_red[32];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // virtual rows of the launch: the matrix's rows, or with several matrices their tile-padded concatenation
    const int vrows = ((EXT & kExtSeg) && p.n_seg > 1) ? kTileRows * p.seg_tile0[p.n_seg] : p.N;
    // This CTA's share of the launch's units (whole tiles when n_tiles_total > 0, else rows): the
    // first split_r CTAs have split_q + 1 of them, the others split_q.
    const int cta = (int)blockIdx.x;
    const int unit_first = cta * p.split_q + min(cta, p.split_r), unit_count = p.split_q + (cta < p.split_r ? 1 : 0);
    const int row_begin = p.n_tiles_total > 0 ? min(vrows, TR * unit_first) : unit_first;
    const int row_end = p.n_tiles_total > 0 ? min(vrows, TR * (unit_first + unit_count)) : unit_first + unit_count;
    const int n_tiles = (row_end - row_begin + TR - 1) / TR;
    const int stage_bytes = TR * p.row_stride;
    const uint64_t wait_limit = p.wait_limit_us ? (uint64_t)p.wait_limit_us * 1000ull : kWaitLimitNs;
    TRACE_STAMP(tid == 0, 0);

    constexpr int kConsumers = kConsumerWarps * NG;
    // Each producer warp sets up its own pipeline's barriers and goes straight on to its first weight
    // copies; the consumers meet the producers' arrival on named barrier 2 before they touch a barrier.
    if (warp >= kConsumers) {
        const int pg = warp - kConsumers;
        if (lane == 0) abort_flag = 0;  // every producer writes the same value, long before any wait can run out
        for (int i = lane; i < p.n_stages * (kConsumerWarps + 1); i += 32) {
            const int st = i / (kConsumerWarps + 1), j = i - st * (kConsumerWarps + 1);
            if (j < kConsumerWarps) mbar_init(smem_u32(&bar_full[pg][st][j]), 1);
            else mbar_init(smem_u32(&bar_empty[pg][st]), kConsumerWarps);
        }
        fence_mbar_init();
        __syncwarp();
        asm volatile("bar.arrive 2, %0;" ::"n"((kConsumers + NG) * 32) : "memory");
    } else {
        asm volatile("bar.sync 2, %0;" ::"n"((kConsumers + NG) * 32) : "memory");
    }
    grid_dep_launch();
    TRACE_STAMP(tid == 0, 1);

    if (warp >= kConsumers) {
        // ---- producer of pipeline g: weights do not depend on the stream-ordered
        // predecessor, so the copies start before griddepcontrol.wait
        const int g = warp - kConsumers;
        const uint32_t ring = sbase + (uint32_t)(p.off_stage + g * p.n_stages * stage_bytes);
        int slot = 0;
        uint32_t phase = 0;
        bool met = !p.step_fill;  // whether this warp has been to named barrier 3 (see below)
        for (int tile = g; tile < n_tiles; tile += NG) {
            const TileRef tr = tile_ref<EXT>(p, row_begin + tile * TR);
            const int row0 = tr.row0;
            const int nrows = min(min(TR, row_end - (row_begin + tile * TR)), tr.N - row0);
            for (int slice = 0; slice < (kLean ? 1 : p.n_slices); ++slice) {
                if (!wait_or_abort(smem_u32(&bar_empty[g][slot]), phase ^ 1, &abort_flag, p.status, kDevTimeoutEmpty, wait_limit)) {
                    if (!met) asm volatile("bar.sync 3, %0;" ::"n"((kConsumers + NG) * 32) : "memory");
                    return;
                }
                const int c0 = slice * p.slice_chunks;
                const int nch = min(p.slice_chunks, p.chunks_per_row - c0);
                const uint32_t bytes = (uint32_t)nch * Chunk<FMT>::bytes;
                const uint32_t full = smem_u32(&bar_full[g][slot][0]);
                if (!split_full) {
                    if (lane == 0) mbar_arrive_expect_tx(full, bytes * (uint32_t)nrows);
                } else if (lane < kConsumerWarps) {
                    // rows of consumer warp `lane` in this tile: its pair, and with 32-row tiles a second pair
                    int cnt = min(max(nrows - 2 * lane, 0), 2);
                    if (RP == 2) cnt += min(max(nrows - 2 * (lane + kConsumerWarps), 0), 2);
                    mbar_arrive_expect_tx(full + 8u * lane, bytes * (uint32_t)cnt);  // no rows: a plain arrival
                }
                __syncwarp();
                if (lane < nrows) {
                    const uint8_t* src = (((EXT & kExtSwiglu) && p.W_up) ? (((lane & 1) ? p.W_up : tr.W) + (size_t)((row0 + lane) >> 1) * p.row_bytes)
                                                          : (tr.W + (size_t)(row0 + lane) * p.row_bytes)) +
                                         (size_t)c0 * Chunk<FMT>::bytes;
                    bulk_g2s(ring + slot * stage_bytes + lane * p.row_stride, src, bytes,
                             split_full ? full + 8u * ((lane >> 1) & (kConsumerWarps - 1)) : full);
                }
                TRACE_STAMP(g == 0 && lane == 0 && tile == 0 && slice == 0, 7);
                // Copies in flight share the SM's ingest rate with the activation loads: with the whole
                // ring requested at once the activations (which every item needs) arrive last. So only
                // the first stage goes out ahead of them; the rest follows once the consumers are about
                // to issue their loads (named barrier 3: they arrive, the producers wait).
                if (!met) {
                    met = true;
                    asm volatile("bar.sync 3, %0;" ::"n"((kConsumers + NG) * 32) : "memory");
                }
                if (++slot == p.n_stages) {
                    slot = 0;
                    phase ^= 1;
                }
            }
        }
        // every producer warp meets barrier 3 exactly once, with or without tiles of its own
        if (!met) asm volatile("bar.sync 3, %0;" ::"n"((kConsumers + NG) * 32) : "memory");
        TRACE_STAMP(g == 0 && lane == 0, 8);
        return;
    }

    // ---- consumers
    grid_dep_wait();  // activations (and Y) belong to the stream-ordered predecessor
    TRACE_STAMP(tid == 0, 2);
    if (p.step_fill) asm volatile("bar.arrive 3, %0;" ::"n"((kConsumers + NG) * 32) : "memory");
    // launch counter of the sharded form: stable while this launch runs (only its last CTA bumps it)
    const unsigned int sh_epoch = ((EXT & kExtShard) && p.sh_world > 0) ? *(volatile unsigned int*)&p.sh_state[1] : 0u;
    const unsigned int sh_buf = (sh_epoch + 1u) & 1u;
    // calls of the candidate form so far, this one included (likewise stable while the launch runs)
    const unsigned int sh_cc = ((EXT & kExtShard) && p.sh_world > 0 && p.sh_topk > 0) ? *(volatile unsigned int*)&p.sh_state[2] + 1u : 0u;
    if ((EXT & kExtNorm) && MT == 1 && p.norm_gamma) stage_x16_norm<FMT>(p, sbase, tid, kConsumers * 32, norm_red);
    else stage_x16<FMT, (EXT & kExtLean) != 0>(p, sbase, tid, kConsumers * 32);
    TRACE_STAMP(tid == 0, 3);
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumers * 32) : "memory");

    const XAddr xa = {sbase + (uint32_t)p.off_xhi, sbase + (uint32_t)p.off_xlo, sbase + (uint32_t)p.off_sxhi, p.K >> 7, p.K};
    constexpr int kGroupsPerChunk = Chunk<FMT>::elems / 128;
    const int g = warp / kConsumerWarps, wl = warp % kConsumerWarps;
    const uint32_t ring = sbase + (uint32_t)(p.off_stage + g * p.n_stages * stage_bytes);
    bool live = true;
    int slot = 0;
    uint32_t phase = 0;
    // Deferred reduction (see the end of the tile loop): sums of the up to three tiles before the current one.
    constexpr bool kDefer = MT == 1 && RP == 1 && !(EXT & kExtSwiglu);
    float hold[3][2] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
    // greedy form of the sharded head: the best (value, global row) among the rows this thread has stored
    float top_v = __int_as_float(0xff800000);
    int top_i = 0x7fffffff;
    int held = 0;
    float acc[RP][2][MT];
#pragma unroll
    for (int pi = 0; pi < RP; ++pi)
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[pi][r][m] = 0.f;

    for (int tile = g; tile < n_tiles; tile += NG) {
        const TileRef tr = tile_ref<EXT>(p, row_begin + tile * TR);
        const int row0 = tr.row0;
        const int nrows = min(min(TR, row_end - (row_begin + tile * TR)), tr.N - row0);
        for (int slice = 0; slice < (kLean ? 1 : p.n_slices); ++slice) {
            if (live) {
                // keep the decision warp-uniform
                const bool ok = wait_or_abort(smem_u32(&bar_full[g][slot][split_full ? wl : 0]), phase, &abort_flag, p.status, kDevTimeoutFull, wait_limit);
                live = __all_sync(0xffffffffu, ok);
            }
            TRACE_STAMP(tid == 0 && tile == 0 && slice == 0, 4);
            if (live && 2 * wl < nrows) {
                const int c0 = slice * p.slice_chunks;
                const int nch = min(p.slice_chunks, p.chunks_per_row - c0);
                const int ng = nch * kGroupsPerChunk, g0 = c0 * kGroupsPerChunk;
                // pair pi of this warp: rows 2 * (wl + 8 pi) and the next one; a pair past the end of
                // the tile re-reads the warp's first pair and its sums are dropped; a tile with an
                // odd row count has no second row for its last pair: reuse the first
                uint32_t rowA[RP], rowB[RP];
#pragma unroll
                for (int pi = 0; pi < RP; ++pi) {
                    const int r0 = 2 * (wl + kConsumerWarps * pi);
                    const int ra = r0 < nrows ? r0 : 2 * wl;
                    rowA[pi] = ring + (uint32_t)(slot * stage_bytes + ra * p.row_stride);
                    rowB[pi] = (ra + 1 < nrows) ? rowA[pi] + (uint32_t)p.row_stride : rowA[pi];
                }
                if constexpr (FMT == kQ6_K || FMT == kQ6_KP) {
                    // half-group units: lanes 0..15 take H = 0 of sixteen groups, lanes 16..31 H = 1
                    for (int gi = (lane & 15); gi < ng; gi += 16) {
#pragma unroll
                        for (int pi = 0; pi < RP; ++pi) {
                            if constexpr (FMT == kQ6_K) item_q6k_half<MT>(rowA[pi], rowB[pi], gi, lane >> 4, g0 + gi, xa, acc[pi]);
                            else item_q6kp_half<MT>(rowA[pi], rowB[pi], gi, lane >> 4, g0 + gi, xa, acc[pi]);
                        }
                    }
                } else {
                    // (half-group units were measured for Q4_K as well: its items are cheap enough that
                    // the second header decode per group costs more than the finer stages give back)
                    for (int gi = lane; gi < ng; gi += 32) {
#pragma unroll
                        for (int pi = 0; pi < RP; ++pi) {
                            if constexpr (FMT == kQ4_K && MT == 1) item_q4k<MT>(rowA[pi], rowB[pi], gi, g0 + gi, xa, acc[pi]);
                            else if constexpr (FMT == kQ4_K) item_q4k_rows<MT>(rowA[pi], rowB[pi], gi, g0 + gi, xa, acc[pi]);
                            else item_q8_0<MT>(rowA[pi], rowB[pi], gi, g0 + gi, xa, acc[pi]);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_empty[g][slot]));
            if (++slot == p.n_stages) {
                slot = 0;
                phase ^= 1;
            }
        }
        if constexpr (kDefer) {
            // One activation row, one row pair per warp: the lanes' partial sums of up to four tiles are
            // kept and reduced together - nine shuffles for eight rows instead of five per tile, and
            // no tile waits for its own reduction before the warp turns to the next one. Same butterfly
            // (xor 16, 8, 4, 2, 1), hence the same bits as the per-tile form below.
            if (++held < 4 && tile + NG < n_tiles) {
                hold[2][0] = hold[1][0]; hold[2][1] = hold[1][1];
                hold[1][0] = hold[0][0]; hold[1][1] = hold[0][1];
                hold[0][0] = acc[0][0][0]; hold[0][1] = acc[0][1][0];
            } else {
                const float v[8] = {hold[2][0], hold[2][1], hold[1][0], hold[1][1], hold[0][0], hold[0][1], acc[0][0][0], acc[0][1][0]};
                const bool h16 = (lane & 16) != 0, h8 = (lane & 8) != 0, h4 = (lane & 4) != 0;
                float w4[4], w2[2];
#pragma unroll
                for (int i = 0; i < 4; ++i) w4[i] = (h16 ? v[4 + i] : v[i]) + __shfl_xor_sync(0xffffffffu, h16 ? v[i] : v[4 + i], 16);
#pragma unroll
                for (int i = 0; i < 2; ++i) w2[i] = (h8 ? w4[2 + i] : w4[i]) + __shfl_xor_sync(0xffffffffu, h8 ? w4[i] : w4[2 + i], 8);
                float s = (h4 ? w2[1] : w2[0]) + __shfl_xor_sync(0xffffffffu, h4 ? w2[0] : w2[1], 4);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                const int o = (h16 ? 4 : 0) + (h8 ? 2 : 0) + (h4 ? 1 : 0), age = 3 - (o >> 1);  // tiles ago; row of the pair: o & 1
                if ((lane & 3) == 0 && age < held && !*(volatile int*)&abort_flag) {
                    const int vr = row_begin + (tile - age * NG) * TR;
                    const TileRef t2 = tile_ref<EXT>(p, vr);
                    const int nr = min(min(TR, row_end - vr), t2.N - t2.row0), rr = 2 * wl + (o & 1);
                    if (rr < nr) {
                        const int n = t2.row0 + rr;
                        if (!kLean && t2.bias) {
                            if (p.x_dtype == B200Q_DT_F32) s += static_cast<const float*>(t2.bias)[n];
                            else if (p.x_dtype == B200Q_DT_F16) s += __half2float(static_cast<const __half*>(t2.bias)[n]);
                            else s += __bfloat162float(static_cast<const __nv_bfloat16*>(t2.bias)[n]);
                        }
                        if ((EXT & kExtShard) && p.sh_world > 0) {
                            p.sh_out[p.sh_rank][(size_t)sh_buf * p.sh_total + (size_t)(p.sh_row_offset + n)] = s;
                            if (cand_before(s, p.sh_row_offset + n, top_v, top_i)) { top_v = s; top_i = p.sh_row_offset + n; }
                        }
                        else if (kLean || p.y_dtype == B200Q_DT_F32) static_cast<float*>(t2.Y)[n] = s;
                        else if (p.y_dtype == B200Q_DT_F16) static_cast<__half*>(t2.Y)[n] = __float2half_rn(s);
                        else static_cast<__nv_bfloat16*>(t2.Y)[n] = __float2bfloat16_rn(s);
                    }
                }
                held = 0;
                hold[0][0] = hold[0][1] = hold[1][0] = hold[1][1] = hold[2][0] = hold[2][1] = 0.f;
            }
            acc[0][0][0] = acc[0][1][0] = 0.f;
            continue;
        }
        // the rows' partial sums live in this warp's lanes: lanes 0..15 finish the first
        // row of the pair, lanes 16..31 the second (five shuffles for both), then write
#pragma unroll
        for (int pi = 0; pi < RP; ++pi) {
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const bool up = lane >= 16;
                float s = (up ? acc[pi][1][m] : acc[pi][0][m]) + __shfl_xor_sync(0xffffffffu, up ? acc[pi][0][m] : acc[pi][1][m], 16);
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                acc[pi][0][m] = acc[pi][1][m] = 0.f;
                const int rr = 2 * (wl + kConsumerWarps * pi) + (up ? 1 : 0);
                if ((EXT & kExtSwiglu) && p.W_up) {
                    // lanes 0..15 hold the gate row's sum, lanes 16..31 the up row's
                    const float u = __shfl_xor_sync(0xffffffffu, s, 16);
                    if (lane == 0 && rr < nrows && m == 0 && !*(volatile int*)&abort_flag) {
                        const float v = s / (1.0f + expf(-s)) * u;  // silu(gate) * up
                        const size_t o = (size_t)((row0 + rr) >> 1);
                        if (p.y_dtype == B200Q_DT_F32) static_cast<float*>(tr.Y)[o] = v;
                        else if (p.y_dtype == B200Q_DT_F16) static_cast<__half*>(tr.Y)[o] = __float2half_rn(v);
                        else static_cast<__nv_bfloat16*>(tr.Y)[o] = __float2bfloat16_rn(v);
                    }
                    continue;
                }
                if ((lane & 15) == 0 && rr < nrows && m < p.M && !*(volatile int*)&abort_flag) {
                    const int n = row0 + rr;
                    if (tr.bias) {
                        if (p.x_dtype == B200Q_DT_F32) s += static_cast<const float*>(tr.bias)[n];
                        else if (p.x_dtype == B200Q_DT_F16) s += __half2float(static_cast<const __half*>(tr.bias)[n]);
                        else s += __bfloat162float(static_cast<const __nv_bfloat16*>(tr.bias)[n]);
                    }
                    const size_t o = (size_t)m * tr.N + n;
                    if ((EXT & kExtShard) && p.sh_world > 0) {
                        // sharded output: into this rank's own result vector first (which of the two
                        // vectors is this launch's parity); the CTA forwards its rows to the peers below
                        p.sh_out[p.sh_rank][(size_t)sh_buf * p.sh_total + (size_t)(p.sh_row_offset + n)] = s;
                        if (m == 0 && cand_before(s, p.sh_row_offset + n, top_v, top_i)) { top_v = s; top_i = p.sh_row_offset + n; }
                    } else if (p.y_dtype == B200Q_DT_F32) static_cast<float*>(tr.Y)[o] = s;
                    else if (p.y_dtype == B200Q_DT_F16) static_cast<__half*>(tr.Y)[o] = __float2half_rn(s);
                    else static_cast<__nv_bfloat16*>(tr.Y)[o] = __float2bfloat16_rn(s);
                }
            }
        }
    }
    TRACE_STAMP((tid & 31) == 0, 5 + (warp >= kConsumerWarps ? 1 : 0));  // last writer of each pipeline wins: about its end
    if ((EXT & kExtShard) && p.sh_world > 0) shard_publish(p, row_begin, row_end, sh_epoch, sh_buf, tid, kConsumers * 32, reinterpret_cast<uint32_t*>(smem_raw + (sbase - smem_u32(smem_raw))), top_v, top_i, sh_cc);
}

// ---- host side ------------------------------------------------------------------------

static int g_opt_groups = 2;
// Q6_K: per-warp full barriers pay while the first and last stage are a visible part of a
// pipeline's stream; beyond this many stages per pipeline one barrier per stage is as fast or faster.
constexpr int kSplitFullMaxStages = 16;
// 0: by shape; 1: 16-row tiles; 2: prefer one pipeline with two row pairs per warp (32-row tiles)
static int g_opt_tile_pairs = 0;
void dp_set_tile_pairs(int v) { g_opt_tile_pairs = v == 2 ? 2 : (v == 1 ? 1 : 0); }
int dp_get_tile_pairs() { return g_opt_tile_pairs; }
// -1: by stream length; 0: one full barrier per stage; 1: one per consumer warp and stage
static int g_opt_split_full = -1;
void dp_set_split_full(int v) { g_opt_split_full = v < 0 ? -1 : (v ? 1 : 0); }
void dp_set_groups(int v) { g_opt_groups = v < 1 ? 1 : (v > 2 ? 2 : v); }
int dp_get_groups() { return g_opt_groups; }
// Bound of the kernels' mbarrier and peer-arrival waits in microseconds; 0: one second.
// 1: launches that qualify take the lean instantiation (kExtLean)
static int g_opt_step_fill = 1;
void dp_set_step_fill(int v) { g_opt_step_fill = v ? 1 : 0; }
static int g_opt_lean = 1;
void dp_set_lean(int v) { g_opt_lean = v ? 1 : 0; }

static int g_opt_wait_limit_us = 0;
void dp_set_wait_limit_us(int v) { g_opt_wait_limit_us = v < 0 ? 0 : v; }
int dp_get_wait_limit_us() { return g_opt_wait_limit_us; }
#ifdef B200Q_TRACE
static unsigned long long* g_trace_buf = nullptr;
static int g_trace_cap = 0, g_trace_idx = 0;
constexpr int kTraceCtas = 160;
// Trace builds only: the next `launches` GEMV launches write their stamps to buf[launch][160 CTAs][16].
extern "C" void b200q_trace_set(void* buf, int launches) {
    g_trace_buf = static_cast<unsigned long long*>(buf);
    g_trace_cap = launches;
    g_trace_idx = 0;
}
// The record of the next traced launch (nullptr when tracing is off or used up).
unsigned long long* dp_trace_next(int grid) {
    return (g_trace_buf && g_trace_idx < g_trace_cap && grid <= kTraceCtas) ? g_trace_buf + (size_t)(g_trace_idx++) * kTraceCtas * 16 : nullptr;
}
#endif

// p.n_stages is the ring depth of ONE pipeline; `ng` pipelines share the shared memory.
template <int FMT>
static bool plan_dp(int M, int N, int K, int sms, size_t smem_max, int ng, int rp, StreamParams& p, int& grid, size_t& smem) {
    const int tile_rows = kTileRows * rp;
    if (K % Chunk<FMT>::elems != 0 || M > 4) return false;
    p.M = M; p.N = N; p.K = K;
    p.row_bytes = (K / Blk<FMT>::elems) * Blk<FMT>::bytes;
    p.chunks_per_row = K / Chunk<FMT>::elems;
    size_t off = 0;
    p.off_xhi = (int)off; off += ((size_t)kXGroupStride * (K / 128) * M + 127) & ~size_t(127);  // int16 activations
    p.off_xlo = (int)off; off += (((size_t)4 * (K / 128) * M) + 127) & ~size_t(127);            // per-group 2^-e
    const size_t sums = FMT == kQ4_K ? (size_t)4 * (K / 32) * M : (FMT == kQ6_K || FMT == kQ6_KP) ? (size_t)4 * (K / 16) * M : 0;
    p.off_sxhi = (int)off; off += (sums + 127) & ~size_t(127);
    p.off_sxlo = p.off_red = (int)off;
    p.off_stage = (int)off;
    if (off + 128 + 4096 > smem_max) return false;
    const size_t avail = smem_max - off - 128;
    // A lane works on one 128-element group, so a slice should hold a multiple of 32
    // groups per row: take the largest such slice whose stage is within the target
    // (at least 32 groups when the row has them), then as many stages as fit.
    constexpr int gpc = Chunk<FMT>::elems / 128;  // groups per chunk: 2 (Q4_K, Q8_0) or 16 (Q6_K)
    const int cpr = p.chunks_per_row;
    const size_t target = (size_t)stream_get_option(2) * 1024;
    int want = stream_get_option(0);
    want = want < 2 ? 2 : (want > kMaxStages ? kMaxStages : want);
    int best = 0;
    constexpr int glanes = (FMT == kQ6_K || FMT == kQ6_KP) ? 16 : 32;  // groups that keep a warp's 32 lanes busy (Q6_K: half-group units)
    for (int sc = 1; sc <= cpr; ++sc) {
        const int groups = sc * gpc;
        if (groups % glanes != 0 && sc != cpr && groups < glanes) continue;
        int rs = sc * Chunk<FMT>::bytes;
        if (rp == 1) rs += ((16 - (rs % 128)) + 128) % 128;
        const size_t sb = (size_t)tile_rows * rs;
        if (sb * 2 * ng > avail) break;
        if (best && sb > target) break;
        if (groups % glanes == 0 || sc == cpr) best = sc;
        else if (!best) best = sc;
    }
    if (!best) return false;
    p.slice_chunks = best;
    p.row_stride = best * Chunk<FMT>::bytes;
    // 16-row tiles: rows padded to 16 (mod 128). 32-row tiles go unpadded - all lanes of a warp read
    // the same row pair, so the row start does not decide bank conflicts - and a third stage fits.
    if (rp == 1) p.row_stride += ((16 - (p.row_stride % 128)) + 128) % 128;
    p.n_slices = (cpr + best - 1) / best;
    const size_t sb = (size_t)tile_rows * p.row_stride;
    int ns = (int)(avail / (sb * ng));
    if (ns > want) ns = want;
    if (ns < 2) return false;
    grid = stream_get_option(3) > 0 ? stream_get_option(3) : sms;
    if (grid > N) grid = N;
    // A pipeline works through its tiles in rounds of one 16-row tile, and a round costs about
    // the same whether the tile is full or not. With at least one tile per SM, give every CTA
    // whole tiles and pick, among grids of 3/4 .. 1 x the SM count, the one with the fewest
    // rounds and then the least idle tile slots: 128 CTAs x 7 tiles beat 148 CTAs x 6.05.
    p.n_tiles_total = 0;
    const int tiles_total = (N + tile_rows - 1) / tile_rows;
    if (stream_get_option(3) <= 0 && M == 1 && tiles_total >= sms) {  // more rows are compute-bound: every SM counts
        long long best_cost = -1;
        for (int gsz = sms; gsz >= (3 * sms) / 4; --gsz) {
            const int per = (tiles_total + gsz - 1) / gsz;
            const int rounds = (per + ng - 1) / ng;
            const long long cost = (long long)rounds * 1000000 + ((long long)gsz * per - tiles_total);
            if (best_cost < 0 || cost < best_cost) { best_cost = cost; grid = gsz; }
        }
        p.n_tiles_total = tiles_total;
    }
    // a ring deeper than the stages a pipeline will ever see only takes shared memory
    // away from the next kernel, which under programmatic dependent launch can move in
    // beside this one and prefetch its weights
    const int rows_per_cta = (N + grid - 1) / grid;
    const int tiles = (rows_per_cta + tile_rows - 1) / tile_rows;
    const int stages_seen = ((tiles + ng - 1) / ng) * p.n_slices;
    if (ns > stages_seen) ns = stages_seen < 1 ? 1 : stages_seen;
    p.n_stages = ns;
    // measured on B200: Q4_K and Q8_0 gain at every stream length (14336 x 4096 Q4_K 8.75 -> 8.0 us,
    // 128256 x 4096 48.5 -> 46.5 us); Q6_K gains on short whole-row streams only
    // (the option only reaches Q6_K: the other formats' kernels are compiled with the split form alone)
    p.split_full = g_opt_split_full >= 0 ? g_opt_split_full
                   : (FMT != kQ6_K && FMT != kQ6_KP) ? 1
                                         : (p.n_slices == 1 && stages_seen <= kSplitFullMaxStages ? 1 : 0);
    smem = off + (size_t)ns * ng * sb + 128;
    return true;
}

template <int FMT, int MT, int NG, int RP, int EXT = 0>
static int launch_dp_k(const StreamParams& p_in, int grid, size_t smem, cudaStream_t st) {
    auto kern = gemv_dp_kernel<FMT, MT, NG, RP, EXT>;
    StreamParams p = p_in;
    {
        const int vrows = ((EXT & kExtSeg) && p.n_seg > 1) ? kTileRows * p.seg_tile0[p.n_seg] : p.N;
        const int units = p.n_tiles_total > 0 ? p.n_tiles_total : vrows;
        p.split_q = units / grid;
        p.split_r = units % grid;
    }
    p.wait_limit_us = (unsigned int)g_opt_wait_limit_us;
    p.step_fill = g_opt_step_fill;
#ifdef B200Q_TRACE
    p.trace = dp_trace_next(grid);
#endif
    static bool configured[64] = {};
    int dev = 0;
    B200Q_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        B200Q_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 2048));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((kConsumerWarps + 1) * NG * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = stream_get_option(1) ? 1 : 0;
    B200Q_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, p));
    return B200Q_OK;
}

template <int FMT, int MT>
static int launch_dp_g(const StreamParams& p, int ng, int rp, int grid, size_t smem, cudaStream_t st) {
    if constexpr (MT == 1) {
        // grouped, sharded and fused forms: one activation row, 16-row tiles
        const int ext = (p.n_seg > 1 ? kExtSeg : 0) | (p.sh_world > 0 ? kExtShard : 0) | (p.norm_gamma ? (kExtNorm | kExtSeg) : 0) |
                        (p.W_up ? kExtSwiglu : 0);
        if (ext == 0 && rp == 1 && g_opt_lean && p.x_dtype == B200Q_DT_F32 && p.y_dtype == B200Q_DT_F32 && !p.bias && p.n_slices == 1 &&
            p.split_full && (p.K >> 3) <= kConsumerWarps * ng * 32)
            return ng == 2 ? launch_dp_k<FMT, 1, 2, 1, kExtLean>(p, grid, smem, st) : launch_dp_k<FMT, 1, 1, 1, kExtLean>(p, grid, smem, st);
        switch (ext) {
            case 0: break;
            case kExtSeg:
                return ng == 2 ? launch_dp_k<FMT, 1, 2, 1, kExtSeg>(p, grid, smem, st) : launch_dp_k<FMT, 1, 1, 1, kExtSeg>(p, grid, smem, st);
            case kExtShard:
                return ng == 2 ? launch_dp_k<FMT, 1, 2, 1, kExtShard>(p, grid, smem, st) : launch_dp_k<FMT, 1, 1, 1, kExtShard>(p, grid, smem, st);
            case kExtNorm | kExtSeg:
                return ng == 2 ? launch_dp_k<FMT, 1, 2, 1, kExtNorm | kExtSeg>(p, grid, smem, st)
                               : launch_dp_k<FMT, 1, 1, 1, kExtNorm | kExtSeg>(p, grid, smem, st);
            case kExtSwiglu:
                return ng == 2 ? launch_dp_k<FMT, 1, 2, 1, kExtSwiglu>(p, grid, smem, st) : launch_dp_k<FMT, 1, 1, 1, kExtSwiglu>(p, grid, smem, st);
            default: return fail(B200Q_ERR_UNSUPPORTED, "gemv: this combination of grouped / sharded / fused forms (%d) is not built", ext);
        }
    }
    if (ng == 2) return launch_dp_k<FMT, MT, 2, 1>(p, grid, smem, st);
    return rp == 2 ? launch_dp_k<FMT, MT, 1, 2>(p, grid, smem, st) : launch_dp_k<FMT, MT, 1, 1>(p, grid, smem, st);
}


template <int FMT>
static int launch_dp_f(const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype, int M, int N,
                       int K, int sms, size_t smem_max, int* status, cudaStream_t st, bool* taken, const ShardOut* sh) {
    StreamParams p = {};
    int grid = 0;
    size_t smem = 0;
    // Candidates in order of preference: one pipeline with 32-row tiles (tile height option 2),
    // two pipelines with 16-row tiles, one pipeline with 16-row tiles.
    int ng = g_opt_groups, rp = 1;
    *taken = false;
    // Measured on B200: with two pipelines of 16-row tiles available, 32-row tiles in one pipeline
    // make no difference (Q4_K, Q8_0) or lose (Q6_K in half-group units: LM head 94 % vs 70 % of
    // the HBM copy rate), so they are only taken on request.
    const bool tall = g_opt_tile_pairs == 2;
    if (tall && !sh && N >= 32 * sms / 2) {
        ng = 1; rp = 2;
        *taken = plan_dp<FMT>(M, N, K, sms, smem_max, ng, rp, p, grid, smem);
    }
    if (!*taken) {
        ng = g_opt_groups; rp = 1;
        *taken = plan_dp<FMT>(M, N, K, sms, smem_max, ng, rp, p, grid, smem);
    }
    if (!*taken && ng == 2) {  // two pipelines do not fit: one
        ng = 1;
        *taken = plan_dp<FMT>(M, N, K, sms, smem_max, ng, rp, p, grid, smem);
    }
    if (!*taken) return B200Q_OK;
    p.W = static_cast<const uint8_t*>(W);
    p.X = X;
    p.bias = bias;
    p.Y = Y;
    p.status = status;
    p.x_dtype = x_dtype;
    p.y_dtype = y_dtype;
    if (sh) {
        p.sh_world = sh->world;
        p.sh_rank = sh->rank;
        p.sh_row_offset = sh->row_offset;
        p.sh_total = sh->total_rows;
        for (int q = 0; q < sh->world; ++q) {
            p.sh_out[q] = sh->out[q];
            p.sh_cand[q] = sh->cand ? sh->cand[q] : nullptr;
        }
        p.sh_state = sh->state;
        p.sh_topk = sh->topk;
        // the candidate form keeps a CTA's rows in registers (four per consumer thread) when k > 1, has
        // kShardSlots CTA slots per rank in the tables, and with k > 1 pools every received candidate in
        // shared memory (the launch asks for that much if its ring is smaller)
        const int threads = kConsumerWarps * ng * 32;
        if (sh->topk > 1 && smem < 2048 + (size_t)sh->world * kShardSlots * sh->topk * 8) smem = 2048 + (size_t)sh->world * kShardSlots * sh->topk * 8;
        if (sh->topk > 0 && ((sh->topk > 1 && (N + grid - 1) / grid + kTileRows > 4 * threads) || grid > kShardSlots))
            return fail(B200Q_ERR_UNSUPPORTED, "gemv_shard_topk: %d rows over %d CTAs exceed the candidate form's capacity", N, grid);
        p.sh_top_val = sh->top_val;
        p.sh_top_idx = sh->top_idx;
    }
    switch (M) {
        case 1: return launch_dp_g<FMT, 1>(p, ng, rp, grid, smem, st);
        case 2: return launch_dp_g<FMT, 2>(p, ng, rp, grid, smem, st);
        case 3: return launch_dp_g<FMT, 3>(p, ng, rp, grid, smem, st);
        default: return launch_dp_g<FMT, 4>(p, ng, rp, grid, smem, st);
    }
}

// Launches the integer-dot-product kernel when the shape qualifies (*taken = true).
int launch_gemv_dp(int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype, int M,
                   int N, int K, int sms, size_t smem_max, int* status, cudaStream_t st, bool* taken, const ShardOut* sh) {
    *taken = false;
    if ((reinterpret_cast<uintptr_t>(W) & 15) != 0) return B200Q_OK;  // bulk copies need 16-byte aligned rows
    smem_max -= 1024;  // the kernel's barriers are static shared memory
    switch (fmt) {
        case kQ4_K: return launch_dp_f<kQ4_K>(W, X, x_dtype, bias, Y, y_dtype, M, N, K, sms, smem_max, status, st, taken, sh);
        case kQ6_K: return launch_dp_f<kQ6_K>(W, X, x_dtype, bias, Y, y_dtype, M, N, K, sms, smem_max, status, st, taken, sh);
        case kQ6_KP: return launch_dp_f<kQ6_KP>(W, X, x_dtype, bias, Y, y_dtype, M, N, K, sms, smem_max, status, st, taken, sh);
        case kQ8_0: return launch_dp_f<kQ8_0>(W, X, x_dtype, bias, Y, y_dtype, M, N, K, sms, smem_max, status, st, taken, sh);
    }
    return fail(B200Q_ERR_BAD_ARG, "gemv: unknown block format %d", fmt);
}

// Gate and up projection with the SwiGLU gate applied in the epilogue: one launch over the two
// matrices' interleaved rows instead of two GEMVs and an elementwise kernel.
template <int FMT>
static int launch_dp_swiglu_f(const void* Wg, const void* Wu, const void* X, int x_dtype, void* Y, int y_dtype, int N, int K,
                              int sms, size_t smem_max, int* status, cudaStream_t st, bool* taken) {
    StreamParams p = {};
    int grid = 0, ng = g_opt_groups;
    size_t smem = 0;
    const int vrows = 2 * N;
    *taken = plan_dp<FMT>(1, vrows, K, sms, smem_max, ng, 1, p, grid, smem);
    if (!*taken && ng == 2) {
        ng = 1;
        *taken = plan_dp<FMT>(1, vrows, K, sms, smem_max, ng, 1, p, grid, smem);
    }
    if (!*taken) return B200Q_OK;
    if (p.n_tiles_total == 0) {  // whole tiles per CTA, so that every CTA starts on a gate row
        p.n_tiles_total = (vrows + kTileRows - 1) / kTileRows;
        if (grid > p.n_tiles_total) grid = p.n_tiles_total;
    }
    p.W = static_cast<const uint8_t*>(Wg);
    p.W_up = static_cast<const uint8_t*>(Wu);
    p.X = X;
    p.Y = Y;
    p.status = status;
    p.x_dtype = x_dtype;
    p.y_dtype = y_dtype;
    return launch_dp_g<FMT, 1>(p, ng, 1, grid, smem, st);
}

int launch_gemv_dp_swiglu(int fmt, const void* Wg, const void* Wu, const void* X, int x_dtype, void* Y, int y_dtype, int N, int K,
                          int sms, size_t smem_max, int* status, cudaStream_t st, bool* taken) {
    *taken = false;
    if (((reinterpret_cast<uintptr_t>(Wg) | reinterpret_cast<uintptr_t>(Wu)) & 15) != 0) return B200Q_OK;
    smem_max -= 1024;  // the kernel's barriers are static shared memory
    switch (fmt) {
        case kQ4_K: return launch_dp_swiglu_f<kQ4_K>(Wg, Wu, X, x_dtype, Y, y_dtype, N, K, sms, smem_max, status, st, taken);
        case kQ6_K: return launch_dp_swiglu_f<kQ6_K>(Wg, Wu, X, x_dtype, Y, y_dtype, N, K, sms, smem_max, status, st, taken);
        case kQ6_KP: return launch_dp_swiglu_f<kQ6_KP>(Wg, Wu, X, x_dtype, Y, y_dtype, N, K, sms, smem_max, status, st, taken);
        case kQ8_0: return launch_dp_swiglu_f<kQ8_0>(Wg, Wu, X, x_dtype, Y, y_dtype, N, K, sms, smem_max, status, st, taken);
    }
    return fail(B200Q_ERR_BAD_ARG, "gemv_swiglu: unknown block format %d", fmt);
}

// Several matrices of one format and K against one activation vector (M = 1) in one launch: the
// fixed cost of a decode GEMV launch (a few microseconds) is paid once for q/k/v or gate/up.
template <int FMT>
static int launch_dp_multi_f(int n_seg, const void* const* W, const int* N, void* const* Y, const void* const* bias, const void* X,
                             int x_dtype, int y_dtype, int K, int sms, size_t smem_max, int* status, cudaStream_t st, bool* taken,
                             const void* gamma, float eps) {
    StreamParams p = {};
    p.norm_gamma = gamma;
    p.norm_eps = eps;
    int tiles = 0;
    for (int s = 0; s < n_seg; ++s) {
        p.seg_tile0[s] = tiles;
        p.seg_rows[s] = N[s];
        p.seg_W[s] = static_cast<const uint8_t*>(W[s]);
        p.seg_Y[s] = Y[s];
        p.seg_bias[s] = bias ? bias[s] : nullptr;
        tiles += (N[s] + kTileRows - 1) / kTileRows;
    }
    p.seg_tile0[n_seg] = tiles;
    int grid = 0, ng = g_opt_groups;
    size_t smem = 0;
    *taken = plan_dp<FMT>(1, kTileRows * tiles, K, sms, smem_max, ng, 1, p, grid, smem);
    if (!*taken && ng == 2) {
        ng = 1;
        *taken = plan_dp<FMT>(1, kTileRows * tiles, K, sms, smem_max, ng, 1, p, grid, smem);
    }
    if (!*taken) return B200Q_OK;
    if (p.n_tiles_total == 0) {  // fewer tiles than SMs: still whole tiles per CTA, so that no tile spans two matrices
        p.n_tiles_total = tiles;
        if (grid > tiles) grid = tiles;
    }
    p.n_seg = n_seg;
    if (n_seg == 1) p.N = N[0];  // one matrix: its own row count, not the tile-padded one
    p.W = p.seg_W[0];
    p.Y = p.seg_Y[0];
    p.bias = p.seg_bias[0];
    p.X = X;
    p.status = status;
    p.x_dtype = x_dtype;
    p.y_dtype = y_dtype;
    return launch_dp_g<FMT, 1>(p, ng, 1, grid, smem, st);
}

int launch_gemv_dp_multi(int fmt, int n_seg, const void* const* W, const int* N, void* const* Y, const void* const* bias,
                         const void* X, int x_dtype, int y_dtype, int K, int sms, size_t smem_max, int* status, cudaStream_t st,
                         bool* taken, const void* gamma, float eps) {
    *taken = false;
    for (int s = 0; s < n_seg; ++s)
        if ((reinterpret_cast<uintptr_t>(W[s]) & 15) != 0) return B200Q_OK;
    smem_max -= 1024;  // the kernel's barriers are static shared memory
    switch (fmt) {
        case kQ4_K: return launch_dp_multi_f<kQ4_K>(n_seg, W, N, Y, bias, X, x_dtype, y_dtype, K, sms, smem_max, status, st, taken, gamma, eps);
        case kQ6_K: return launch_dp_multi_f<kQ6_K>(n_seg, W, N, Y, bias, X, x_dtype, y_dtype, K, sms, smem_max, status, st, taken, gamma, eps);
        case kQ6_KP: return launch_dp_multi_f<kQ6_KP>(n_seg, W, N, Y, bias, X, x_dtype, y_dtype, K, sms, smem_max, status, st, taken, gamma, eps);
        case kQ8_0: return launch_dp_multi_f<kQ8_0>(n_seg, W, N, Y, bias, X, x_dtype, y_dtype, K, sms, smem_max, status, st, taken, gamma, eps);
    }
    return fail(B200Q_ERR_BAD_ARG, "gemv_multi: unknown block format %d", fmt);
}

}  // namespace b200q

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

namespace b200q {

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

// Staged activations: group gg of row m is 16 segments of eight int16 (256 bytes);
// segment i sits at position i ^ (gg & 7), so lanes working on consecutive groups read
// the same segment number from different banks. All shared-memory traffic below goes
// through explicit ld.shared / st.shared with 32-bit shared addresses.
template <int FMT, typename XT>
__device__ __forceinline__ void stage_x16(const StreamParams& p, uint32_t sbase, int tid) {
    const XT* X = static_cast<const XT*>(p.X);
    const int segs = p.K >> 3, groups = p.K >> 7;
    const int total = segs * p.M;  // K % 256 == 0, so a multiple of 32
    for (int idx = tid; idx < total; idx += kConsumerThreads) {
        const int m = idx / segs, seg = idx - m * segs;
        const int gg = seg >> 4, i = seg & 15;
        float v[8];
        if constexpr (sizeof(XT) == 4) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(X + (size_t)m * p.K) + 2 * seg);
            const float4 b = __ldg(reinterpret_cast<const float4*>(X + (size_t)m * p.K) + 2 * seg + 1);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
            v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
            union {
                uint4 q;
                XT h[8];
            } pk;
            pk.q = __ldg(reinterpret_cast<const uint4*>(X + (size_t)m * p.K) + seg);
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = to_f32<XT>(pk.h[k]);
        }
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
        sts128(sbase + p.off_xhi + (uint32_t)((m * groups + gg) * 256 + ((i ^ (gg & 7)) << 4)), o);
        if (i == 0) sts32(sbase + p.off_xlo + (uint32_t)(m * groups + gg) * 4, (uint32_t)(127 - e) << 23);
        if constexpr (FMT == kQ4_K) {  // sums over 32 elements = 4 segments
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if ((i & 3) == 0) sts32(sbase + p.off_sxhi + (uint32_t)(m * (p.K >> 5) + (seg >> 2)) * 4, (uint32_t)sum);
        } else if constexpr (FMT == kQ6_K) {  // sums over 16 elements = 2 segments
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            if ((i & 1) == 0) sts32(sbase + p.off_sxhi + (uint32_t)(m * (p.K >> 4) + (seg >> 1)) * 4, (uint32_t)sum);
        }
    }
}

// Shared-memory addresses an item needs for the staged activations.
struct XAddr {
    uint32_t x16, xsc, sxi;  // region bases (x16 256-byte aligned)
    int groups, K;
};
// Address of segment `I` of group gg, row m: xg = base of the group XOR-ed with the rotation.
template <int I>
__device__ __forceinline__ uint4 x_seg(uint32_t xg) { return lds128i<0>(xg ^ (uint32_t)(I << 4)); }

// ---- one item = one 128-element group of two weight rows ---------------------------
// rowA/rowB: shared addresses of this stage's bytes of the two rows; gi: group index
// inside the stage; gg: group index along the whole row; acc[r][m]: FP32 partial sums.

template <int MT>
__device__ __forceinline__ void item_q4k(uint32_t rowA, uint32_t rowB, int gi, int gg, const XAddr& xa,
                                         float (&acc)[2][MT]) {
    const int b = gi >> 1, hb = gi & 1;
    const uint32_t pr[2] = {rowA + (uint32_t)b * 144u, rowB + (uint32_t)b * 144u};
    uint32_t scw[2], mw[2];
    float d[2], dm[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint4 h = lds128i<0>(pr[r]);
        // the four 6-bit scales / mins of sub-blocks 4*hb .. 4*hb+3, one per byte
        const uint32_t sclo = h.y & 0x3f3f3f3fu, schi = (h.w & 0x0f0f0f0fu) | ((h.y >> 2) & 0x30303030u);
        const uint32_t mlo = h.z & 0x3f3f3f3fu, mhi = ((h.w >> 4) & 0x0f0f0f0fu) | ((h.z >> 2) & 0x30303030u);
        scw[r] = hb ? schi : sclo;
        mw[r] = hb ? mhi : mlo;
        d[r] = h2f(h.x & 0xFFFFu);
        dm[r] = h2f(h.x >> 16);
    }
    const uint32_t qa[2] = {pr[0] + 64u * hb, pr[1] + 64u * hb};
    int isum[2][MT];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) isum[r][m] = 0;
#pragma unroll
    for (int c2 = 0; c2 < 2; ++c2) {
        // 32 bytes of quants per row: low nibbles = sub-block 2*c2, high nibbles = 2*c2+1
        uint32_t lo[2][8], hi[2][8];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint4 q0 = c2 ? lds128i<48>(qa[r]) : lds128i<16>(qa[r]);
            const uint4 q1 = c2 ? lds128i<64>(qa[r]) : lds128i<32>(qa[r]);
            const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                lo[r][k] = w[k] & 0x0F0F0F0Fu;
                hi[r][k] = (w[k] >> 4) & 0x0F0F0F0Fu;
            }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const uint32_t xg = xa.x16 + (uint32_t)((m * xa.groups + gg) * 256 + ((gg & 7) << 4));
            uint4 xl[4], xh[4];  // segments 8*c2+0..3 (low-nibble sub-block), 8*c2+4..7 (high-nibble)
            if (c2 == 0) {
                xl[0] = x_seg<0>(xg); xl[1] = x_seg<1>(xg); xl[2] = x_seg<2>(xg); xl[3] = x_seg<3>(xg);
                xh[0] = x_seg<4>(xg); xh[1] = x_seg<5>(xg); xh[2] = x_seg<6>(xg); xh[3] = x_seg<7>(xg);
            } else {
                xl[0] = x_seg<8>(xg); xl[1] = x_seg<9>(xg); xl[2] = x_seg<10>(xg); xl[3] = x_seg<11>(xg);
                xh[0] = x_seg<12>(xg); xh[1] = x_seg<13>(xg); xh[2] = x_seg<14>(xg); xh[3] = x_seg<15>(xg);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                int cl = 0, ch = 0;
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    cl = dp2a_lo_su(xl[s].x, lo[r][2 * s], cl);
                    cl = dp2a_hi_su(xl[s].y, lo[r][2 * s], cl);
                    cl = dp2a_lo_su(xl[s].z, lo[r][2 * s + 1], cl);
                    cl = dp2a_hi_su(xl[s].w, lo[r][2 * s + 1], cl);
                    ch = dp2a_lo_su(xh[s].x, hi[r][2 * s], ch);
                    ch = dp2a_hi_su(xh[s].y, hi[r][2 * s], ch);
                    ch = dp2a_lo_su(xh[s].z, hi[r][2 * s + 1], ch);
                    ch = dp2a_hi_su(xh[s].w, hi[r][2 * s + 1], ch);
                }
                // |sc * c| <= 63 * 32*15*16383 = 4.95e8 and four of them fit an int32
                isum[r][m] += (int)((scw[r] >> (16 * c2)) & 0xFFu) * cl + (int)((scw[r] >> (16 * c2 + 8)) & 0xFFu) * ch;
            }
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
__device__ __forceinline__ void q8_block_words(uint32_t base, float& d, uint32_t (&qs)[8]) {
    // block J of the group starts at 34*J: 4-byte aligned for even J, 2 (mod 4) for odd J
    constexpr int O = (J & 1) ? 34 * J - 2 : 34 * J;
    const uint32_t w[9] = {lds32i<O>(base),      lds32i<O + 4>(base),  lds32i<O + 8>(base),
                           lds32i<O + 12>(base), lds32i<O + 16>(base), lds32i<O + 20>(base),
                           lds32i<O + 24>(base), lds32i<O + 28>(base), lds32i<O + 32>(base)};
    if (J & 1) {
        d = h2f(w[0] >> 16);
#pragma unroll
        for (int k = 0; k < 8; ++k) qs[k] = w[k + 1];
    } else {
        d = h2f(w[0] & 0xFFFFu);
#pragma unroll
        for (int k = 0; k < 8; ++k) qs[k] = __byte_perm(w[k], w[k + 1], 0x5432);
    }
}

template <int MT, int J>
__device__ __forceinline__ void q8_block(const uint32_t (&pr)[2], int gg, const XAddr& xa, float (&acc)[2][MT]) {
    uint32_t qs[2][8];
    float d[2];
    q8_block_words<J>(pr[0], d[0], qs[0]);
    q8_block_words<J>(pr[1], d[1], qs[1]);
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const uint32_t xg = xa.x16 + (uint32_t)((m * xa.groups + gg) * 256 + ((gg & 7) << 4));
        const uint4 xv[4] = {x_seg<4 * J>(xg), x_seg<4 * J + 1>(xg), x_seg<4 * J + 2>(xg), x_seg<4 * J + 3>(xg)};
        const float xs = __uint_as_float(lds32i<0>(xa.xsc + (uint32_t)(m * xa.groups + gg) * 4u));
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            int c = 0;
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                c = dp2a_lo_ss(xv[s].x, qs[r][2 * s], c);
                c = dp2a_hi_ss(xv[s].y, qs[r][2 * s], c);
                c = dp2a_lo_ss(xv[s].z, qs[r][2 * s + 1], c);
                c = dp2a_hi_ss(xv[s].w, qs[r][2 * s + 1], c);
            }
            acc[r][m] = fmaf(d[r] * xs, (float)c, acc[r][m]);
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
__device__ __forceinline__ void funnel_words(uint32_t a, uint32_t sh, uint32_t* out) {
    // out[k] = bytes 4k .. 4k+3 of the stream that starts sh/8 bytes after `a`
    if constexpr (K0 < N) {
        out[K0] = __funnelshift_r(lds32i<4 * K0>(a), lds32i<4 * K0 + 4>(a), sh);
        funnel_words<N, K0 + 1>(a, sh, out);
    }
}

template <int MT, int H, int Q>
__device__ __forceinline__ void q6_sub(const uint32_t (&ql)[2][16], const uint32_t (&qh)[2][8],
                                       const uint32_t (&su)[2][2], int gg, const XAddr& xa, float (&accg)[2][MT]) {
    // sub-block (Q, H): 16 elements at 32*Q + 16*H of the group, raw6 = nibble | two qh bits << 4
    uint32_t v[2][4];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const uint32_t a = ql[r][4 * H + 8 * (Q & 1) + w], hb = qh[r][4 * H + w];
            const uint32_t nib = (Q < 2 ? a : (a >> 4)) & 0x0F0F0F0Fu;
            const uint32_t h2 = (Q == 0 ? hb << 4 : Q == 1 ? hb << 2 : Q == 2 ? hb : hb >> 2) & 0x30303030u;
            v[r][w] = nib | h2;
        }
    constexpr int SI = 2 * Q + H;  // scale byte and 16-element sum index inside the group
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const uint32_t xg = xa.x16 + (uint32_t)((m * xa.groups + gg) * 256 + ((gg & 7) << 4));
        const uint4 x0 = x_seg<4 * Q + 2 * H>(xg), x1 = x_seg<4 * Q + 2 * H + 1>(xg);
        const int sx = (int)lds32i<4 * SI>(xa.sxi + (uint32_t)(m * (xa.K >> 4) + gg * 8) * 4u);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            int c = 0;
            c = dp2a_lo_su(x0.x, v[r][0], c);
            c = dp2a_hi_su(x0.y, v[r][0], c);
            c = dp2a_lo_su(x0.z, v[r][1], c);
            c = dp2a_hi_su(x0.w, v[r][1], c);
            c = dp2a_lo_su(x1.x, v[r][2], c);
            c = dp2a_hi_su(x1.y, v[r][2], c);
            c = dp2a_lo_su(x1.z, v[r][3], c);
            c = dp2a_hi_su(x1.w, v[r][3], c);
            // sum (raw6 - 32) * x = c - 32 * sum x
            accg[r][m] = fmaf(biased_s8_to_f32(su[r][SI >> 2], SI & 3), (float)(c - 32 * sx), accg[r][m]);
        }
    }
}

template <int MT>
__device__ __forceinline__ void item_q6k(uint32_t rowA, uint32_t rowB, int gi, int gg, const XAddr& xa,
                                         float (&acc)[2][MT]) {
    const int bi = gi >> 1, G = gi & 1;
    // blocks are 210 bytes: odd blocks of a 16-byte aligned chunk start at 2 (mod 4). Read
    // aligned words from 2 bytes earlier and funnel-shift; for even blocks the shift is 0.
    const uint32_t sh = (uint32_t)(bi & 1) * 16u;
    uint32_t ql[2][16], qh[2][8], su[2][2];
    float d[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint32_t L = (r ? rowB : rowA) + (uint32_t)(bi * 210 - (bi & 1) * 2);
        funnel_words<16>(L + 64u * G, sh, ql[r]);
        funnel_words<8>(L + 128u + 32u * G, sh, qh[r]);
        funnel_words<2>(L + 192u + 8u * G, sh, su[r]);
        su[r][0] ^= 0x80808080u;
        su[r][1] ^= 0x80808080u;
        d[r] = h2f((lds32i<208>(L) >> sh) & 0xFFFFu);
    }
    float accg[2][MT];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) accg[r][m] = 0.f;
    q6_sub<MT, 0, 0>(ql, qh, su, gg, xa, accg);
    q6_sub<MT, 0, 1>(ql, qh, su, gg, xa, accg);
    q6_sub<MT, 0, 2>(ql, qh, su, gg, xa, accg);
    q6_sub<MT, 0, 3>(ql, qh, su, gg, xa, accg);
    q6_sub<MT, 1, 0>(ql, qh, su, gg, xa, accg);
    q6_sub<MT, 1, 1>(ql, qh, su, gg, xa, accg);
    q6_sub<MT, 1, 2>(ql, qh, su, gg, xa, accg);
    q6_sub<MT, 1, 3>(ql, qh, su, gg, xa, accg);
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const float xs = __uint_as_float(lds32i<0>(xa.xsc + (uint32_t)(m * xa.groups + gg) * 4u));
#pragma unroll
        for (int r = 0; r < 2; ++r) acc[r][m] = fmaf(d[r] * xs, accg[r][m], acc[r][m]);
    }
}

template <int FMT, int MT>
__global__ void __launch_bounds__(kStreamThreads, 1) gemv_dp_kernel(const StreamParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 255u) & ~255u;  // shared-space address, 256-byte aligned
    __shared__ uint64_t bar_full[kMaxStages];
    __shared__ uint64_t bar_empty[kMaxStages];
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = gridDim.x;
    const int row_begin = (int)((long long)p.N * blockIdx.x / G);
    const int row_end = (int)((long long)p.N * (blockIdx.x + 1) / G);
    const int n_tiles = (row_end - row_begin + kTileRows - 1) / kTileRows;
    const int total_iters = n_tiles * p.n_slices;
    const int stage_bytes = kTileRows * p.row_stride;

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < p.n_stages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), kConsumerWarps);
        }
        fence_mbar_init();
    }
    __syncthreads();
    grid_dep_launch();

    if (warp == kConsumerWarps) {
        stream_producer<FMT>(p, sbase, bar_full, bar_empty, &abort_flag, row_begin, row_end, total_iters, lane);
        return;
    }

    grid_dep_wait();  // activations (and Y) belong to the stream-ordered predecessor
    if (p.x_dtype == B200Q_DT_F32) stage_x16<FMT, float>(p, sbase, tid);
    else if (p.x_dtype == B200Q_DT_F16) stage_x16<FMT, __half>(p, sbase, tid);
    else stage_x16<FMT, __nv_bfloat16>(p, sbase, tid);
    consumer_bar_sync();

    const XAddr xa = {sbase + (uint32_t)p.off_xhi, sbase + (uint32_t)p.off_xlo, sbase + (uint32_t)p.off_sxhi, p.K >> 7, p.K};
    constexpr int kGroupsPerChunk = Chunk<FMT>::elems / 128;
    bool live = true;
    float acc[2][MT];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;

    for (int it = 0; it < total_iters; ++it) {
        const int slot = it % p.n_stages;
        const int tile = it / p.n_slices, slice = it - tile * p.n_slices;
        const int row0 = row_begin + tile * kTileRows;
        const int nrows = min(kTileRows, row_end - row0);
        if (live) {
            const bool ok = wait_or_abort(smem_u32(&bar_full[slot]), (it / p.n_stages) & 1, &abort_flag, p.status, kDevTimeoutFull);
            live = __all_sync(0xffffffffu, ok);
        }
        if (live && 2 * warp < nrows) {
            const int c0 = slice * p.slice_chunks;
            const int nch = min(p.slice_chunks, p.chunks_per_row - c0);
            const int ng = nch * kGroupsPerChunk, g0 = c0 * kGroupsPerChunk;
            const uint32_t rowA = sbase + (uint32_t)(p.off_stage + slot * stage_bytes + (2 * warp) * p.row_stride);
            // a tile with an odd row count has no second row for its last pair: reuse the first
            const uint32_t rowB = (2 * warp + 1 < nrows) ? rowA + (uint32_t)p.row_stride : rowA;
            for (int gi = lane; gi < ng; gi += 32) {
                if constexpr (FMT == kQ4_K) item_q4k<MT>(rowA, rowB, gi, g0 + gi, xa, acc);
                else if constexpr (FMT == kQ8_0) item_q8_0<MT>(rowA, rowB, gi, g0 + gi, xa, acc);
                else item_q6k<MT>(rowA, rowB, gi, g0 + gi, xa, acc);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_empty[slot]));

        if (slice == p.n_slices - 1) {
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    float s = acc[r][m];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                    acc[r][m] = 0.f;
                    const int rr = 2 * warp + r;
                    if (lane == 0 && rr < nrows && m < p.M && !*(volatile int*)&abort_flag) {
                        const int n = row0 + rr;
                        if (p.bias) {
                            if (p.x_dtype == B200Q_DT_F32) s += static_cast<const float*>(p.bias)[n];
                            else if (p.x_dtype == B200Q_DT_F16) s += __half2float(static_cast<const __half*>(p.bias)[n]);
                            else s += __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[n]);
                        }
                        const size_t o = (size_t)m * p.N + n;
                        if (p.y_dtype == B200Q_DT_F32) static_cast<float*>(p.Y)[o] = s;
                        else if (p.y_dtype == B200Q_DT_F16) static_cast<__half*>(p.Y)[o] = __float2half_rn(s);
                        else static_cast<__nv_bfloat16*>(p.Y)[o] = __float2bfloat16_rn(s);
                    }
                }
        }
    }
}

// ---- host side ------------------------------------------------------------------------

template <int FMT>
static bool plan_dp(int M, int N, int K, int sms, size_t smem_max, StreamParams& p, int& grid, size_t& smem) {
    if (K % Chunk<FMT>::elems != 0 || M > 4) return false;
    p.M = M; p.N = N; p.K = K;
    p.row_bytes = (K / Blk<FMT>::elems) * Blk<FMT>::bytes;
    p.chunks_per_row = K / Chunk<FMT>::elems;
    size_t off = 0;
    p.off_xhi = (int)off; off += (size_t)2 * K * M;                     // int16 activations (multiple of 256)
    p.off_xlo = (int)off; off += (((size_t)4 * (K / 128) * M) + 127) & ~size_t(127);  // per-group 2^-e
    const size_t sums = FMT == kQ4_K ? (size_t)4 * (K / 32) * M : FMT == kQ6_K ? (size_t)4 * (K / 16) * M : 0;
    p.off_sxhi = (int)off; off += (sums + 127) & ~size_t(127);
    p.off_sxlo = p.off_red = (int)off;
    p.off_stage = (int)off;
    if (off + 256 + 4096 > smem_max) return false;
    // Q4_K lanes read 16-byte vectors at a 144-byte stride, Q8_0 8-byte ... at 136: any
    // row stride works for the lanes of one row; pad rows to 16 (mod 128) to spread the
    // two rows of a pair.
    if (!plan_ring<FMT>(p, smem_max - off - 256, (size_t)stream_get_option(2) * 1024, stream_get_option(0), 16))
        return false;
    smem = off + (size_t)p.n_stages * kTileRows * p.row_stride + 256;
    grid = stream_get_option(3) > 0 ? stream_get_option(3) : sms;
    if (grid > N) grid = N;
    return true;
}

template <int FMT, int MT>
static int launch_dp_k(const StreamParams& p, int grid, size_t smem, cudaStream_t st) {
    auto kern = gemv_dp_kernel<FMT, MT>;
    static bool configured[64] = {};
    int dev = 0;
    B200Q_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        B200Q_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 1024));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kStreamThreads);
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

template <int FMT>
static int launch_dp_f(const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype, int M, int N,
                       int K, int sms, size_t smem_max, int* status, cudaStream_t st, bool* taken) {
    StreamParams p = {};
    int grid = 0;
    size_t smem = 0;
    *taken = plan_dp<FMT>(M, N, K, sms, smem_max, p, grid, smem);
    if (!*taken) return B200Q_OK;
    p.W = static_cast<const uint8_t*>(W);
    p.X = X;
    p.bias = bias;
    p.Y = Y;
    p.status = status;
    p.x_dtype = x_dtype;
    p.y_dtype = y_dtype;
    switch (M) {
        case 1: return launch_dp_k<FMT, 1>(p, grid, smem, st);
        case 2: return launch_dp_k<FMT, 2>(p, grid, smem, st);
        case 3: return launch_dp_k<FMT, 3>(p, grid, smem, st);
        default: return launch_dp_k<FMT, 4>(p, grid, smem, st);
    }
}

// Launches the integer-dot-product kernel when the shape qualifies (*taken = true).
int launch_gemv_dp(int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype, int M,
                   int N, int K, int sms, size_t smem_max, int* status, cudaStream_t st, bool* taken) {
    *taken = false;
    if ((reinterpret_cast<uintptr_t>(W) & 15) != 0) return B200Q_OK;  // bulk copies need 16-byte aligned rows
    switch (fmt) {
        case kQ4_K: return launch_dp_f<kQ4_K>(W, X, x_dtype, bias, Y, y_dtype, M, N, K, sms, smem_max, status, st, taken);
        case kQ6_K: return launch_dp_f<kQ6_K>(W, X, x_dtype, bias, Y, y_dtype, M, N, K, sms, smem_max, status, st, taken);
        case kQ8_0: return launch_dp_f<kQ8_0>(W, X, x_dtype, bias, Y, y_dtype, M, N, K, sms, smem_max, status, st, taken);
    }
    return fail(B200Q_ERR_BAD_ARG, "gemv: unknown block format %d", fmt);
}

}  // namespace b200q

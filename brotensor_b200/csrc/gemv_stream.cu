// Streaming decode GEMV for sm_100a: Y(M,N) = X(M,K) * decode(W(N,K))^T (+bias), M <= 8.
//
// The kernel is built to be HBM-bound:
//   * a persistent grid of one CTA per SM; CTA c owns the contiguous row range
//     [N*c/G, N*(c+1)/G), i.e. one contiguous byte range of the weight;
//   * a producer warp streams that range through a ring of shared-memory stages
//     with 1-D bulk async copies (cp.async.bulk + mbarrier complete_tx), one
//     copy per weight row and stage, so tens of KB per SM are always in flight
//     and no register or issue slot is spent on global loads;
//   * eight consumer warps split the K extent of a 16-row tile between them.
//     Quants are unpacked in registers into exact small-integer FP16 values
//     (nibble | 0x6400 is 1024+n; one HFMA2 removes the bias and, for Q4_K,
//     folds the 6-bit sub-block scale in, which stays exact because
//     sc*n <= 945 < 2048) and fed to warp-level m16n8k16 MMAs whose N=8
//     columns are the up-to-8 activation rows; block scales are applied to the
//     FP32 accumulators. Activations are staged once per CTA as FP16 hi (+lo)
//     halves already in MMA fragment order, so every weight byte is read from
//     HBM exactly once whatever M is;
//   * partial sums of the eight warps are combined through shared memory, bias
//     is added and Y written; only shuffles-free smem traffic, no atomics, and
//     the summation order is fixed, so results are deterministic.
// Weight prefetch starts before griddepcontrol.wait, so under programmatic
// dependent launch the next GEMV's weights stream in while the previous kernel
// drains. Every wait is bounded: when one runs out the kernel records a code in
// the device status word, stops computing and returns normally.
//
// Takes the place of brotensor's linear_q4k_fp16_gemv_kernel
// (src/cuda/q4k.cu:159-224), linear_q6k_fp16_gemv_kernel (q6k.cu:117-176) and
// linear_q8_0_fp16_gemv_kernel (q8_0.cu:75-138) plus their host-side widening
// rules (q4k.cu:243-281).
#include "stream_common.cuh"

namespace b200q {

// Slot of (t = k-group owner lane, m = activation row) inside one 4*MG*8-byte page
// of the staged activations; chosen so a warp's B-fragment loads hit distinct banks.
template <int MG>
__device__ __forceinline__ int x_slot(int t, int m) {
    if constexpr (MG == 8) return ((m >> 2) << 4) + (t << 2) + (m & 3);
    else return t * MG + m;
}

// Where k-group kg (4 consecutive k) of the row lives: page index and owner lane t.
template <int FMT>
__device__ __forceinline__ void x_place(int kg, int& page, int& t) {
    if constexpr (FMT == kQ6_K) {
        page = kg >> 2;  // one page per 16-element sub-block
        t = kg & 3;
    } else {
        page = ((kg >> 3) << 1) + (kg & 1);  // two pages per 32 elements: even / odd k-groups
        t = (kg >> 1) & 3;
    }
}

// ---- activation staging -------------------------------------------------------
// Writes, for every activation row m < M and k-group, the four values as FP16 in
// the order [k0,k2,k1,k3] (hi part, and the FP16 residual as lo part when XSPLIT).
// For Q4_K also the per-32-element sums (needed for the dmin*m term), packed as
// (even sub-block, odd sub-block) half2 pairs.
template <int FMT, int MG, bool XSPLIT, typename XT>
__device__ __forceinline__ void stage_activations(const StreamParams& p, uint8_t* smem, int tid) {
    const XT* X = static_cast<const XT*>(p.X);
    const int kgs = p.K >> 2;
    const int total = kgs * p.M;  // multiple of 64
    for (int idx = tid; idx < total; idx += kConsumerThreads) {
        const int m = idx / kgs, kg = idx - m * kgs;
        float v[4];
        if constexpr (sizeof(XT) == 4) {
            const float4 f = __ldg(reinterpret_cast<const float4*>(X + (size_t)m * p.K) + kg);
            v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
        } else {
            union {
                uint2 q;
                XT h[4];
            } pk;
            pk.q = __ldg(reinterpret_cast<const uint2*>(X + (size_t)m * p.K) + kg);
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] = to_f32<XT>(pk.h[k]);
        }
        __half hi[4], lo[4];
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            hi[k] = __float2half_rn(v[k]);
            const float r = v[k] - __half2float(hi[k]);
            lo[k] = __float2half_rn(r);
            s += XSPLIT ? (__half2float(hi[k]) + __half2float(lo[k])) : __half2float(hi[k]);
        }
        int page, t;
        x_place<FMT>(kg, page, t);
        const int off = (page * 4 * MG + x_slot<MG>(t, m)) * 8;
        union {
            __half h[4];
            uint2 q;
        } o;
        o.h[0] = hi[0]; o.h[1] = hi[2]; o.h[2] = hi[1]; o.h[3] = hi[3];
        *reinterpret_cast<uint2*>(smem + p.off_xhi + off) = o.q;
        if constexpr (XSPLIT) {
            o.h[0] = lo[0]; o.h[1] = lo[2]; o.h[2] = lo[1]; o.h[3] = lo[3];
            *reinterpret_cast<uint2*>(smem + p.off_xlo + off) = o.q;
        }
        if constexpr (FMT == kQ4_K) {
            // eight consecutive lanes hold the eight k-groups of one 32-element sub-block
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            const float s_odd = __shfl_down_sync(0xffffffffu, s, 8);  // next sub-block's sum
            const int sub = kg >> 3;
            if ((kg & 7) == 0 && (sub & 1) == 0) {
                const __half a_hi = __float2half_rn(s), b_hi = __float2half_rn(s_odd);
                const int blk = sub >> 3, tt = (sub & 7) >> 1;
                const int soff = ((blk * 4 + tt) * MG + m) * 4;
                *reinterpret_cast<__half2*>(smem + p.off_sxhi + soff) = __halves2half2(a_hi, b_hi);
                // the sums always carry a residual half: it costs one tiny MMA per block
                const __half a_lo = __float2half_rn(s - __half2float(a_hi));
                const __half b_lo = __float2half_rn(s_odd - __half2float(b_hi));
                *reinterpret_cast<__half2*>(smem + p.off_sxlo + soff) = __halves2half2(a_lo, b_lo);
            }
        }
    }
}

constexpr uint32_t kMagic = 0x64006400u;      // half2(1024, 1024)
constexpr uint32_t kH2_1024n = 0xE400E400u;   // half2(-1024)
constexpr uint32_t kH2_64n = 0xD400D400u;     // half2(-64)
constexpr uint32_t kH2_16th = 0x2C002C00u;    // half2(1/16)
constexpr uint32_t kH2_1152 = 0x64806480u;    // half2(1152) = 1024 + 128
constexpr uint32_t kH2_1056 = 0x64206420u;    // half2(1056) = 1024 + 32
constexpr uint32_t kH2_96n = 0xD600D600u;     // half2(-96)

// ---- per-format work units: 16 rows x 256 elements ------------------------------
// rA / rB: shared-memory byte addresses of rows g and g+8 at the unit's first block.
// kblk: index of the unit's 256-element span along K (for the activation pages).
// acc: the lane's four FP32 accumulators (rows g, g+8 x activation rows 2t, 2t+1).

template <int MG, bool XSPLIT, bool HASB>
__device__ __forceinline__ void unit_q4k(uint32_t rA, uint32_t rB, int kblk, int g, int t, uint32_t xhi, uint32_t xlo,
                                         uint32_t sxhi, uint32_t sxlo, float acc[4]) {
    const bool bact = g < MG;
    const uint32_t xoff = (uint32_t)x_slot<MG>(t, bact ? g : 0) * 8u;
    constexpr uint32_t page = 4 * MG * 8;
    const uint4 hA = lds128(rA);
    uint4 hB = make_uint4(0, 0, 0, 0);
    if constexpr (HASB) hB = lds128(rB);
    // 6-bit scales / mins of all eight sub-blocks, four per word
    const uint32_t scA[2] = {hA.y & 0x3f3f3f3fu, (hA.w & 0x0f0f0f0fu) | ((hA.y >> 2) & 0x30303030u)};
    const uint32_t mnA[2] = {hA.z & 0x3f3f3f3fu, ((hA.w >> 4) & 0x0f0f0f0fu) | ((hA.z >> 2) & 0x30303030u)};
    const uint32_t scB[2] = {hB.y & 0x3f3f3f3fu, (hB.w & 0x0f0f0f0fu) | ((hB.y >> 2) & 0x30303030u)};
    const uint32_t mnB[2] = {hB.z & 0x3f3f3f3fu, ((hB.w >> 4) & 0x0f0f0f0fu) | ((hB.z >> 2) & 0x30303030u)};
    float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const uint2 qA = lds64(rA + 16 + 32 * p + 8 * t);
        uint2 qB = make_uint2(0, 0);
        if constexpr (HASB) qB = lds64(rB + 16 + 32 * p + 8 * t);
        const int b0 = (2 * p) & 3;
        // half2(sc, sc) for the low-nibble (2p) and high-nibble (2p+1) sub-blocks
        const uint32_t slA = hsub2_u32(__byte_perm(scA[p >> 1], 0x64646464u, 0x4040 | (b0 << 8) | b0), kMagic);
        const uint32_t shA = hsub2_u32(__byte_perm(scA[p >> 1], 0x64646464u, 0x4040 | ((b0 + 1) << 8) | (b0 + 1)), kMagic);
        const uint32_t slB = hsub2_u32(__byte_perm(scB[p >> 1], 0x64646464u, 0x4040 | (b0 << 8) | b0), kMagic);
        const uint32_t shB = hsub2_u32(__byte_perm(scB[p >> 1], 0x64646464u, 0x4040 | ((b0 + 1) << 8) | (b0 + 1)), kMagic);
        const uint32_t clA = hmul2_u32(slA, kH2_1024n), clB = hmul2_u32(slB, kH2_1024n);
        const uint32_t khA = hmul2_u32(shA, kH2_16th), khB = hmul2_u32(shB, kH2_16th);
        const uint32_t chA = hmul2_u32(shA, kH2_64n), chB = hmul2_u32(shB, kH2_64n);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const uint32_t wA = j ? qA.y : qA.x, wB = j ? qB.y : qB.x;
            const uint32_t wA8 = wA >> 8, wB8 = wB >> 8;
            // (1024+n)*sc - 1024*sc and (1024+16n)*(sc/16) - 64*sc: both exactly n*sc
            const uint32_t l02A = hfma2_u32(lop3_and_or(wA, 0x000F000Fu, kMagic), slA, clA);
            const uint32_t l13A = hfma2_u32(lop3_and_or(wA8, 0x000F000Fu, kMagic), slA, clA);
            const uint32_t h02A = hfma2_u32(lop3_and_or(wA, 0x00F000F0u, kMagic), khA, chA);
            const uint32_t h13A = hfma2_u32(lop3_and_or(wA8, 0x00F000F0u, kMagic), khA, chA);
            uint32_t l02B = 0, l13B = 0, h02B = 0, h13B = 0;
            if constexpr (HASB) {
                l02B = hfma2_u32(lop3_and_or(wB, 0x000F000Fu, kMagic), slB, clB);
                l13B = hfma2_u32(lop3_and_or(wB8, 0x000F000Fu, kMagic), slB, clB);
                h02B = hfma2_u32(lop3_and_or(wB, 0x00F000F0u, kMagic), khB, chB);
                h13B = hfma2_u32(lop3_and_or(wB8, 0x00F000F0u, kMagic), khB, chB);
            }
            // activation pages: sub-block S = kblk*8 + 2p (+1), k-group 2t+j -> page S*2+j
            const uint32_t pgl = (uint32_t)(((kblk * 8 + 2 * p) * 2 + j)) * page + xoff;
            const uint32_t pgh = pgl + 2 * page;
            uint2 bl = make_uint2(0, 0), bh = make_uint2(0, 0);
            if (bact) {
                bl = lds64(xhi + pgl);
                bh = lds64(xhi + pgh);
            }
            mma16816(c, l02A, l02B, l13A, l13B, bl.x, bl.y);
            mma16816(c, h02A, h02B, h13A, h13B, bh.x, bh.y);
            if constexpr (XSPLIT) {
                uint2 bl2 = make_uint2(0, 0), bh2 = make_uint2(0, 0);
                if (bact) {
                    bl2 = lds64(xlo + pgl);
                    bh2 = lds64(xlo + pgh);
                }
                mma16816(c, l02A, l02B, l13A, l13B, bl2.x, bl2.y);
                mma16816(c, h02A, h02B, h13A, h13B, bh2.x, bh2.y);
            }
        }
    }
    // dmin * sum_sub m[sub] * sum_k x[k]: an m16n8k8 MMA over the eight sub-blocks
    const uint32_t selw = (t & 2) ? 1u : 0u, sh = (t & 1) * 16;
    const uint32_t mA2 = hsub2_u32(__byte_perm((selw ? mnA[1] : mnA[0]) >> sh, 0x64646464u, 0x4140), kMagic);
    uint32_t mB2 = 0;
    if constexpr (HASB) mB2 = hsub2_u32(__byte_perm((selw ? mnB[1] : mnB[0]) >> sh, 0x64646464u, 0x4140), kMagic);
    float cm[4] = {0.f, 0.f, 0.f, 0.f};
    const uint32_t soff = (uint32_t)(((kblk * 4 + t) * MG + (bact ? g : 0)) * 4);
    uint32_t bs = 0;
    if (bact) bs = lds32(sxhi + soff);
    uint32_t bs2 = 0;
    if (bact) bs2 = lds32(sxlo + soff);
    mma1688(cm, mA2, mB2, bs);
    mma1688(cm, mA2, mB2, bs2);
    const float dA = h2f(hA.x & 0xFFFFu), dmA = h2f(hA.x >> 16);
    acc[0] += dA * c[0] - dmA * cm[0];
    acc[1] += dA * c[1] - dmA * cm[1];
    if constexpr (HASB) {
        const float dB = h2f(hB.x & 0xFFFFu), dmB = h2f(hB.x >> 16);
        acc[2] += dB * c[2] - dmB * cm[2];
        acc[3] += dB * c[3] - dmB * cm[3];
    }
}

// 8 bytes at a shared address that is 2 (mod 4) when ODD2, else 4-byte aligned.
template <bool ODD2>
__device__ __forceinline__ uint2 lds8_q(uint32_t a) {
    if constexpr (!ODD2) {
        return make_uint2(lds32(a), lds32(a + 4));
    } else {
        const uint32_t x0 = lds32(a - 2), x1 = lds32(a + 2), x2 = lds32(a + 6);
        return make_uint2(__byte_perm(x0, x1, 0x5432), __byte_perm(x1, x2, 0x5432));
    }
}
template <bool ODD2>
__device__ __forceinline__ uint32_t lds4_q(uint32_t a) {
    if constexpr (!ODD2) return lds32(a);
    else return __byte_perm(lds16(a), lds16(a + 2), 0x5410);
}

template <int MG, bool XSPLIT, bool HASB>
__device__ __forceinline__ void unit_q8_0(uint32_t rA, uint32_t rB, int kblk, int g, int t, uint32_t xhi, uint32_t xlo,
                                          float acc[4]) {
    const bool bact = g < MG;
    const uint32_t xoff = (uint32_t)x_slot<MG>(t, bact ? g : 0) * 8u;
    constexpr uint32_t page = 4 * MG * 8;
#pragma unroll
    for (int jb = 0; jb < 8; ++jb) {
        constexpr int dummy = 0;
        (void)dummy;
        const uint32_t o = 34 * jb;
        const float dA = h2f(lds16(rA + o));
        // (34*jb + 2) % 4 is 2 for even jb, 0 for odd jb (chunk base is 16-byte aligned)
        uint2 qA, qB = make_uint2(0, 0);
        if ((jb & 1) == 0) qA = lds8_q<true>(rA + o + 2 + 8 * t);
        else qA = lds8_q<false>(rA + o + 2 + 8 * t);
        float dB = 0.f;
        if constexpr (HASB) {
            dB = h2f(lds16(rB + o));
            if ((jb & 1) == 0) qB = lds8_q<true>(rB + o + 2 + 8 * t);
            else qB = lds8_q<false>(rB + o + 2 + 8 * t);
        }
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            // int8 q -> byte q+128 -> half 1024+128+q -> subtract 1152: exact
            const uint32_t uA = (j ? qA.y : qA.x) ^ 0x80808080u;
            const uint32_t a02A = hsub2_u32(__byte_perm(uA, 0x64646464u, 0x4240), kH2_1152);
            const uint32_t a13A = hsub2_u32(__byte_perm(uA, 0x64646464u, 0x4341), kH2_1152);
            uint32_t a02B = 0, a13B = 0;
            if constexpr (HASB) {
                const uint32_t uB = (j ? qB.y : qB.x) ^ 0x80808080u;
                a02B = hsub2_u32(__byte_perm(uB, 0x64646464u, 0x4240), kH2_1152);
                a13B = hsub2_u32(__byte_perm(uB, 0x64646464u, 0x4341), kH2_1152);
            }
            const uint32_t pg = (uint32_t)((kblk * 8 + jb) * 2 + j) * page + xoff;
            uint2 b = make_uint2(0, 0);
            if (bact) b = lds64(xhi + pg);
            mma16816(c, a02A, a02B, a13A, a13B, b.x, b.y);
            if constexpr (XSPLIT) {
                uint2 b2 = make_uint2(0, 0);
                if (bact) b2 = lds64(xlo + pg);
                mma16816(c, a02A, a02B, a13A, a13B, b2.x, b2.y);
            }
        }
        acc[0] += dA * c[0];
        acc[1] += dA * c[1];
        if constexpr (HASB) {
            acc[2] += dB * c[2];
            acc[3] += dB * c[3];
        }
    }
}

// int8 scale byte `idx` of word u (already xor 0x80808080) -> exact float
__device__ __forceinline__ float s8_to_f32(uint32_t u, int idx) {
    return __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7440 | idx)) - 8388736.0f;  // 2^23 + 128
}

template <int MG, bool XSPLIT, bool HASB, bool ODD2>
__device__ __forceinline__ void unit_q6k(uint32_t rA, uint32_t rB, int kblk, int g, int t, uint32_t xhi, uint32_t xlo,
                                         float acc[4]) {
    const bool bact = g < MG;
    const uint32_t xoff = (uint32_t)x_slot<MG>(t, bact ? g : 0) * 8u;
    constexpr uint32_t page = 4 * MG * 8;
    float cb[4] = {0.f, 0.f, 0.f, 0.f};  // sum over sub-blocks of sc * (v . x)
#pragma unroll
    for (int G = 0; G < 2; ++G) {
        // the eight int8 scales of this 128-element group, biased to unsigned
        const uint32_t sA0 = lds4_q<ODD2>(rA + 192 + 8 * G) ^ 0x80808080u;
        const uint32_t sA1 = lds4_q<ODD2>(rA + 196 + 8 * G) ^ 0x80808080u;
        uint32_t sB0 = 0, sB1 = 0;
        if constexpr (HASB) {
            sB0 = lds4_q<ODD2>(rB + 192 + 8 * G) ^ 0x80808080u;
            sB1 = lds4_q<ODD2>(rB + 196 + 8 * G) ^ 0x80808080u;
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t o = 64 * G + 16 * h + 4 * t;
            const uint32_t qlA[2] = {lds4_q<ODD2>(rA + o), lds4_q<ODD2>(rA + o + 32)};
            const uint32_t qhA = lds4_q<ODD2>(rA + 128 + 32 * G + 16 * h + 4 * t);
            uint32_t qlB[2] = {0, 0}, qhB = 0;
            if constexpr (HASB) {
                qlB[0] = lds4_q<ODD2>(rB + o);
                qlB[1] = lds4_q<ODD2>(rB + o + 32);
                qhB = lds4_q<ODD2>(rB + 128 + 32 * G + 16 * h + 4 * t);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                // raw6 = nibble | (two qh bits << 4); quads 0,1 use low nibbles, 2,3 high nibbles
                uint32_t a02A, a13A, a02B = 0, a13B = 0;
                const uint32_t srcA = qlA[q & 1], srcB = qlB[q & 1];
                if (q < 2) {
                    const int sl = 4 - 2 * q, sr = 4 + 2 * q;
                    a02A = hsub2_u32(lop3_and_or(qhA << sl, 0x00300030u, lop3_and_or(srcA, 0x000F000Fu, kMagic)), kH2_1056);
                    a13A = hsub2_u32(lop3_and_or(qhA >> sr, 0x00300030u, lop3_and_or(srcA >> 8, 0x000F000Fu, kMagic)), kH2_1056);
                    if constexpr (HASB) {
                        a02B = hsub2_u32(lop3_and_or(qhB << sl, 0x00300030u, lop3_and_or(srcB, 0x000F000Fu, kMagic)), kH2_1056);
                        a13B = hsub2_u32(lop3_and_or(qhB >> sr, 0x00300030u, lop3_and_or(srcB >> 8, 0x000F000Fu, kMagic)), kH2_1056);
                    }
                } else {
                    // keep the high nibble in place: half = 1024 + 16*raw6, then *1/16 - 96 = raw6 - 32
                    const int sl = 8 - 2 * q, sr = 2 * q;
                    a02A = hfma2_u32(lop3_and_or(qhA << sl, 0x03000300u, lop3_and_or(srcA, 0x00F000F0u, kMagic)), kH2_16th, kH2_96n);
                    a13A = hfma2_u32(lop3_and_or(qhA >> sr, 0x03000300u, lop3_and_or(srcA >> 8, 0x00F000F0u, kMagic)), kH2_16th, kH2_96n);
                    if constexpr (HASB) {
                        a02B = hfma2_u32(lop3_and_or(qhB << sl, 0x03000300u, lop3_and_or(srcB, 0x00F000F0u, kMagic)), kH2_16th, kH2_96n);
                        a13B = hfma2_u32(lop3_and_or(qhB >> sr, 0x03000300u, lop3_and_or(srcB >> 8, 0x00F000F0u, kMagic)), kH2_16th, kH2_96n);
                    }
                }
                // 16-element sub-block index along K: kblk*16 + G*8 + q*2 + h
                const uint32_t pg = (uint32_t)(kblk * 16 + G * 8 + q * 2 + h) * page + xoff;
                float c[4] = {0.f, 0.f, 0.f, 0.f};
                uint2 b = make_uint2(0, 0);
                if (bact) b = lds64(xhi + pg);
                mma16816(c, a02A, a02B, a13A, a13B, b.x, b.y);
                if constexpr (XSPLIT) {
                    uint2 b2 = make_uint2(0, 0);
                    if (bact) b2 = lds64(xlo + pg);
                    mma16816(c, a02A, a02B, a13A, a13B, b2.x, b2.y);
                }
                // scale byte index within the group's eight: 2q + h
                const int si = 2 * q + h;
                const float fA = s8_to_f32(si < 4 ? sA0 : sA1, si & 3);
                cb[0] = fmaf(fA, c[0], cb[0]);
                cb[1] = fmaf(fA, c[1], cb[1]);
                if constexpr (HASB) {
                    const float fB = s8_to_f32(si < 4 ? sB0 : sB1, si & 3);
                    cb[2] = fmaf(fB, c[2], cb[2]);
                    cb[3] = fmaf(fB, c[3], cb[3]);
                }
            }
        }
    }
    const float dA = h2f(ODD2 ? lds16(rA + 208) : (lds32(rA + 208) & 0xFFFFu));
    acc[0] = fmaf(dA, cb[0], acc[0]);
    acc[1] = fmaf(dA, cb[1], acc[1]);
    if constexpr (HASB) {
        const float dB = h2f(ODD2 ? lds16(rB + 208) : (lds32(rB + 208) & 0xFFFFu));
        acc[2] = fmaf(dB, cb[2], acc[2]);
        acc[3] = fmaf(dB, cb[3], acc[3]);
    }
}

// One work unit = 16 rows x 256 elements: unit index u inside the stage.
template <int FMT, int MG, bool XSPLIT, bool HASB>
__device__ __forceinline__ void run_unit(uint32_t stage, int row_stride, int u, int kblk, int g, int t, uint32_t xhi,
                                         uint32_t xlo, uint32_t sxhi, uint32_t sxlo, float acc[4]) {
    const uint32_t rA0 = stage + (uint32_t)(g * row_stride);
    const uint32_t rB0 = rA0 + (uint32_t)(8 * row_stride);
    if constexpr (FMT == kQ4_K) {
        unit_q4k<MG, XSPLIT, HASB>(rA0 + u * 144, rB0 + u * 144, kblk, g, t, xhi, xlo, sxhi, sxlo, acc);
    } else if constexpr (FMT == kQ8_0) {
        unit_q8_0<MG, XSPLIT, HASB>(rA0 + u * 272, rB0 + u * 272, kblk, g, t, xhi, xlo, acc);
    } else {
        // block u of the stage; chunks are 16-byte aligned, so odd blocks sit at 2 (mod 4)
        if (u & 1) unit_q6k<MG, XSPLIT, HASB, true>(rA0 + u * 210, rB0 + u * 210, kblk, g, t, xhi, xlo, acc);
        else unit_q6k<MG, XSPLIT, HASB, false>(rA0 + u * 210, rB0 + u * 210, kblk, g, t, xhi, xlo, acc);
    }
}

template <int FMT, int MG, bool XSPLIT>
__global__ void __launch_bounds__(kStreamThreads, 1) gemv_stream_kernel(const StreamParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
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
        stream_producer<FMT>(p, smem_u32(smem), bar_full, bar_empty, &abort_flag, row_begin, row_end, total_iters, lane);
        return;
    }

    // ---- consumers
    grid_dep_wait();  // activations (and Y) belong to the stream-ordered predecessor
    if (p.x_dtype == B200Q_DT_F32) stage_activations<FMT, MG, XSPLIT, float>(p, smem, tid);
    else if (p.x_dtype == B200Q_DT_F16) stage_activations<FMT, MG, XSPLIT, __half>(p, smem, tid);
    else stage_activations<FMT, MG, XSPLIT, __nv_bfloat16>(p, smem, tid);
    consumer_bar_sync();

    const int g = lane >> 2, t = lane & 3;
    const uint32_t xhi = smem_u32(smem + p.off_xhi), xlo = smem_u32(smem + p.off_xlo);
    const uint32_t sxhi = smem_u32(smem + p.off_sxhi), sxlo = smem_u32(smem + p.off_sxlo);
    float* red = reinterpret_cast<float*>(smem + p.off_red);
    bool live = true;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};

    for (int it = 0; it < total_iters; ++it) {
        const int slot = it % p.n_stages;
        const int tile = it / p.n_slices, slice = it - tile * p.n_slices;
        const int row0 = row_begin + tile * kTileRows;
        const int nrows = min(kTileRows, row_end - row0);
        if (live) {
            // keep the decision warp-uniform: the MMAs below need all 32 lanes
            const bool ok = wait_or_abort(smem_u32(&bar_full[slot]), (it / p.n_stages) & 1, &abort_flag, p.status, kDevTimeoutFull);
            live = __all_sync(0xffffffffu, ok);
        }
        if (live) {
            const int c0 = slice * p.slice_chunks;
            const int nch = min(p.slice_chunks, p.chunks_per_row - c0);
            const int n_units = nch * Chunk<FMT>::units;
            const int unit0 = c0 * Chunk<FMT>::units;  // first 256-element span of this stage
            const uint32_t stage = smem_u32(smem + p.off_stage + slot * stage_bytes);
            // spans are dealt round-robin over the warps along the whole row
            int u = (warp - (unit0 % kConsumerWarps) + kConsumerWarps) % kConsumerWarps;
            if (nrows > 8) {
                for (; u < n_units; u += kConsumerWarps)
                    run_unit<FMT, MG, XSPLIT, true>(stage, p.row_stride, u, unit0 + u, g, t, xhi, xlo, sxhi, sxlo, acc);
            } else {
                for (; u < n_units; u += kConsumerWarps)
                    run_unit<FMT, MG, XSPLIT, false>(stage, p.row_stride, u, unit0 + u, g, t, xhi, xlo, sxhi, sxlo, acc);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_empty[slot]));

        if (slice == p.n_slices - 1) {
            // combine the eight warps' partial sums of this row tile
            float* buf = red + (tile & 1) * (kConsumerWarps * 32 * 4);
            reinterpret_cast<float4*>(buf)[warp * 32 + lane] = make_float4(acc[0], acc[1], acc[2], acc[3]);
            acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
            consumer_bar_sync();
            if (tid < 128) {
                const int ln = tid & 31, j = tid >> 5;
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w) s += buf[(w * 32 + ln) * 4 + j];
                const int r = (ln >> 2) + ((j & 2) ? 8 : 0);
                const int m = 2 * (ln & 3) + (j & 1);
                if (r < nrows && m < p.M && !*(volatile int*)&abort_flag) {
                    const int n = row0 + r;
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

// ---- host side ------------------------------------------------------------------

struct StreamPlan {
    StreamParams p;
    int grid;
    size_t smem;
    bool xsplit;
    int mg;
};

static int g_opt_stages = 4;
static int g_opt_pdl = 0;
static int g_opt_stage_kb = 40;
static int g_opt_grid = 0;
void stream_set_option(int which, int value) {
    if (which == 0) g_opt_stages = value;
    else if (which == 1) g_opt_pdl = value;
    else if (which == 2) g_opt_stage_kb = value;
    else g_opt_grid = value;
}
int stream_get_option(int which) {
    return which == 0 ? g_opt_stages : which == 1 ? g_opt_pdl : which == 2 ? g_opt_stage_kb : g_opt_grid;
}

template <int FMT>
static bool plan_stream(int x_dtype, int M, int N, int K, int sms, size_t smem_max, StreamPlan& pl) {
    if (K % Chunk<FMT>::elems != 0) return false;  // rows must be made of 16-byte aligned chunks
    StreamParams& p = pl.p;
    p.M = M; p.N = N; p.K = K;
    p.row_bytes = (K / Blk<FMT>::elems) * Blk<FMT>::bytes;
    p.chunks_per_row = K / Chunk<FMT>::elems;
    pl.mg = M == 1 ? 1 : M == 2 ? 2 : M <= 4 ? 4 : 8;
    const size_t xbytes = (size_t)2 * K * pl.mg;
    const size_t sxbytes = FMT == kQ4_K ? (size_t)(K / 256) * 4 * pl.mg * 4 : 0;
    for (int split = (x_dtype == B200Q_DT_F32) ? 1 : 0; split >= 0; --split) {
        size_t off = 0;
        p.off_xhi = (int)off; off += xbytes;
        p.off_xlo = (int)off; off += split ? xbytes : 0;
        p.off_sxhi = (int)off; off += (sxbytes + 127) & ~size_t(127);
        p.off_sxlo = (int)off; off += (sxbytes + 127) & ~size_t(127);
        p.off_red = (int)off; off += 2 * kConsumerWarps * 32 * 16;
        off = (off + 127) & ~size_t(127);
        p.off_stage = (int)off;
        if (off + 128 + 2 * 1024 > smem_max) continue;
        const size_t avail = smem_max - off - 128;
        // stage = 16 rows x slice; row stride padded to 32 (mod 128) so that the four
        // row quads of a half-warp read distinct banks
        int sc = p.chunks_per_row;
        const int want_stages = g_opt_stages < 2 ? 2 : (g_opt_stages > kMaxStages ? kMaxStages : g_opt_stages);
        for (;;) {
            int rs = sc * Chunk<FMT>::bytes;
            rs += ((32 - (rs % 128)) + 128) % 128;
            const size_t sb = (size_t)kTileRows * rs;
            const size_t target = (size_t)g_opt_stage_kb * 1024;
            int ns = (int)(avail / sb);
            if (ns > want_stages) ns = want_stages;
            if ((sb <= target && ns >= 2) || sc == 1) {
                if (ns < 2) break;
                p.slice_chunks = sc;
                p.row_stride = rs;
                p.n_stages = ns;
                p.n_slices = (p.chunks_per_row + sc - 1) / sc;
                pl.smem = off + (size_t)ns * sb + 128;
                pl.xsplit = split != 0;
                int grid = g_opt_grid > 0 ? g_opt_grid : sms;
                if (grid > N) grid = N;
                pl.grid = grid;
                return true;
            }
            sc = (sc + 1) / 2;
        }
    }
    return false;
}

template <int FMT, int MG, bool XSPLIT>
static int launch_stream_k(const StreamPlan& pl, cudaStream_t st) {
    auto kern = gemv_stream_kernel<FMT, MG, XSPLIT>;
    // raise the dynamic shared-memory limit once per device and instantiation (a
    // racing double call is harmless); later launches, e.g. under stream capture,
    // then make no call besides the launch itself
    static bool configured[64] = {};
    int dev = 0;
    B200Q_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        B200Q_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 1024));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)pl.grid);
    cfg.blockDim = dim3(kStreamThreads);
    cfg.dynamicSmemBytes = pl.smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_opt_pdl ? 1 : 0;
    B200Q_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, pl.p));
    return B200Q_OK;
}

template <int FMT, int MG>
static int launch_stream_x(const StreamPlan& pl, cudaStream_t st) {
    return pl.xsplit ? launch_stream_k<FMT, MG, true>(pl, st) : launch_stream_k<FMT, MG, false>(pl, st);
}

template <int FMT>
static int launch_stream_f(const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype, int M,
                           int N, int K, int sms, size_t smem_max, int* status, cudaStream_t st, bool* taken) {
    StreamPlan pl = {};
    *taken = plan_stream<FMT>(x_dtype, M, N, K, sms, smem_max, pl);
    if (!*taken) return B200Q_OK;
    pl.p.W = static_cast<const uint8_t*>(W);
    pl.p.X = X;
    pl.p.bias = bias;
    pl.p.Y = Y;
    pl.p.status = status;
    pl.p.x_dtype = x_dtype;
    pl.p.y_dtype = y_dtype;
    switch (pl.mg) {
        case 1: return launch_stream_x<FMT, 1>(pl, st);
        case 2: return launch_stream_x<FMT, 2>(pl, st);
        case 4: return launch_stream_x<FMT, 4>(pl, st);
        default: return launch_stream_x<FMT, 8>(pl, st);
    }
}

// Launches the streaming kernel when the shape qualifies (*taken = true); leaves
// *taken = false when the caller has to use the plain-load kernel instead.
int launch_gemv_stream(int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype,
                       int M, int N, int K, int sms, size_t smem_max, int* status, cudaStream_t st, bool* taken) {
    *taken = false;
    if (fmt == kQ6_KP) return B200Q_OK;  // the regrouped Q6_K layout is read by the integer-dot kernel only
    if ((reinterpret_cast<uintptr_t>(W) & 15) != 0) return B200Q_OK;  // bulk copies need 16-byte aligned rows
    switch (fmt) {
        case kQ4_K: return launch_stream_f<kQ4_K>(W, X, x_dtype, bias, Y, y_dtype, M, N, K, sms, smem_max, status, st, taken);
        case kQ6_K: return launch_stream_f<kQ6_K>(W, X, x_dtype, bias, Y, y_dtype, M, N, K, sms, smem_max, status, st, taken);
        case kQ8_0: return launch_stream_f<kQ8_0>(W, X, x_dtype, bias, Y, y_dtype, M, N, K, sms, smem_max, status, st, taken);
    }
    return fail(B200Q_ERR_BAD_ARG, "gemv: unknown block format %d", fmt);
}

}  // namespace b200q

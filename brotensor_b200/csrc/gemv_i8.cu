// Small-batch decode GEMV on the integer tensor cores, Q8_0 and Q4_K, 2..8 activation rows, K = 2048
// or 4096 (sm_100a): Y(M, N) = X(M, K) * decode(W(N, K))^T in little more than the time of ONE activation row.
//
// The dp2a kernel (gemv_dp.cu) does M times the work for M rows and the FP16-MMA streaming kernel
// (gemv_stream.cu) decodes every weight to FP16 first; Q8_0's quants ARE int8, so here they go into
// mma.sync.m16n8k32.s8 as they lie in the GGUF blocks:
//   * A (16 weight rows x 32 k) is one Q8_0 block column of a 16-row tile, read straight from the
//     staged raw bytes (the 34-byte blocks are 2-byte aligned: even blocks take two words and a funnel
//     shift per fragment register, odd blocks one word);
//   * B (32 k x 8 columns) holds the 8 activation rows as int8 planes: x is converted once per launch
//     to 15-bit fixed point with a power-of-two scale per 128-element group (as gemv_dp.cu does),
//     x16 = 128 * hi + lo with hi in -128..127 and lo in 0..127, one MMA per plane; the block's integer
//     dot product 128 * C_hi + C_lo is exact, the block scale d and the group's 2^-e are applied in FP32;
//   * the 16 warps of a CTA split K (warp w owns blocks [w, w + 1) * K / 512 of every row), so a warp's
//     B fragments are the same for every tile and stay in REGISTERS for the whole launch (32 of them at
//     K = 4096) - each warp stages its own slice of x with two shuffles per group, no shared memory
//     and no CTA barrier for the activations;
//   * a tile's 16 rows are 16 bulk copies (one per warp, which refills "its" row itself as soon as the
//     tile's partial sums have met on the CTA barrier) into a ring of three 70 KB stages; rows are
//     padded by 16 bytes in shared memory so that the eight rows a fragment load touches fall into
//     different banks;
//   * the warps' 16 x 8 partial sums are added in a fixed order through shared memory (double
//     buffered, one CTA barrier per tile), so results are reproducible.
// Q4_K goes the same way: a sub-block of 32 weights is one k-step, the low nibbles of a 32-byte run of
// quants are the A fragments of the even sub-block and the high nibbles those of the odd one (two
// aligned words per row and sub-block pair, a mask / shift-and-mask per register), the 6-bit scales
// and mins are applied to the integer sums per 128-element group (four sub-blocks fit an int32), and
// the mins' term dmin * m * sum(x) uses per-sub-block sums of the fixed-point activations that each
// warp computes while it stages its slice.
// Per block column a warp issues two MMAs, six to eight shared loads and about sixteen scalar
// instructions for 16 x 32 x 8 products: 3.2 M warp instructions for 14336 x 4096, a third of the
// time the bytes take - the kernel streams at the M = 1 rate for every M up to 8.
//
// Takes the place of the per-row GEMV loop brotensor's batched Q8_0 op falls back to for B < 4
// (src/cuda/q8_0.cu:261-314) and of its WMMA kernel for 4 <= B <= 8.
#include "dp_common.cuh"

namespace b200q {

constexpr int kI8Warps = 16;
constexpr int kI8TileRows = 16;
constexpr int kI8MaxStages = 5;

struct I8Params {
    const uint8_t* W;
    const void* X;
    const void* bias;
    void* Y;
    int* status;
    int M, N, K;
    int x_dtype, y_dtype;
    int row_bytes, row_stride;  // bytes of a weight row in global memory / in a stage (padded)
    int n_stages;
    int tile_q, tile_r;  // CTA b owns tile_q + (b < tile_r) 16-row tiles, starting at b * tile_q + min(b, tile_r)
    unsigned int wait_limit_us;
};

__device__ __forceinline__ void mma_s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Four consecutive activations of row m starting at element k (k % 4 == 0), as floats.
__device__ __forceinline__ float4 i8_load_x4(const void* X, int x_dtype, int K, int m, int k) {
    if (x_dtype == B200Q_DT_F32) return __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(X) + (size_t)m * K + k));
    const uint2 q = __ldg(reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(X) + (size_t)m * K + k));
    if (x_dtype == B200Q_DT_F16) {
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&q.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&q.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    return make_float4(__uint_as_float(q.x << 16), __uint_as_float(q.x & 0xFFFF0000u), __uint_as_float(q.y << 16),
                       __uint_as_float(q.y & 0xFFFF0000u));
}

// BPW = k-steps of 32 (Q8_0 blocks, Q4_K sub-blocks) per warp: K = 512 * BPW.
// PACK (at most four activation rows): the MMA's eight columns hold BOTH planes - column c < 4 is the hi
// plane of row c, column c + 4 its lo plane - so a k-step is ONE MMA instead of two (the legacy integer
// MMA is what bounds this kernel, not memory). Everything up to the final sum is linear in the
// accumulator, so the two planes' columns are carried separately through scales, mins and the K-split
// reduction and only combined, 128 * hi + lo, when a result is written.
template <int FMT, int BPW, bool PACK>
__global__ void __launch_bounds__(kI8Warps * 32, 1) gemv_i8_kernel(const __grid_constant__ I8Params p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 127u) & ~127u;
    __shared__ uint64_t bar_full[kI8MaxStages];
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int cta = (int)blockIdx.x;
    const int tile_first = cta * p.tile_q + min(cta, p.tile_r), n_tiles = p.tile_q + (cta < p.tile_r ? 1 : 0);
    const uint32_t stage_bytes = (uint32_t)(kI8TileRows * p.row_stride);
    const uint32_t part_base = sbase + (uint32_t)p.n_stages * stage_bytes;  // [2][16 warps][16 rows][8 cols] floats
    const uint64_t wait_limit = p.wait_limit_us ? (uint64_t)p.wait_limit_us * 1000ull : kWaitLimitNs;

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < p.n_stages; ++s) mbar_init(smem_u32(&bar_full[s]), kI8Warps);
        fence_mbar_init();
    }
    __syncthreads();
    // Warp w feeds row w of every tile: one bulk copy, or a plain arrival for a row past the matrix.
    auto feed = [&](int tile, int stage) {
        const int row = kI8TileRows * (tile_first + tile) + warp;
        const uint32_t full = smem_u32(&bar_full[stage]);
        if (row < p.N) {
            mbar_arrive_expect_tx(full, (uint32_t)p.row_bytes);
            bulk_g2s(sbase + (uint32_t)stage * stage_bytes + (uint32_t)(warp * p.row_stride), p.W + (size_t)row * p.row_bytes, (uint32_t)p.row_bytes, full);
        } else {
            mbar_arrive(full);
        }
    };
    // weights do not depend on the stream-ordered predecessor: the first stages go out before griddepcontrol.wait
    if (lane == 0)
        for (int s = 0; s < p.n_stages && s < n_tiles; ++s) feed(s, s);
    grid_dep_launch();
    grid_dep_wait();  // activations (and Y) belong to the predecessor

    // ---- this warp's slice of the activations as B fragments: column g of the MMA is activation row g,
    // the thread holds k = 4t .. 4t+3 and 16+4t .. 16+4t+3 of each of its BPW blocks
    uint32_t xb[BPW][PACK ? 2 : 4];  // [block][hi k 0-15, hi k 16-31, lo k 0-15, lo k 16-31]; PACK: this column's plane only
    float cs[(BPW + 3) / 4][2];   // 2^-e of the block's 128-element group, for the C columns 2t and 2t+1
    int xsum[FMT == kQ4_K ? BPW : 1][2];  // Q4_K: sum of the k-step's 32 fixed-point activations (PACK: of the column's plane), same columns
    const int xrow = PACK ? (g & 3) : g;  // the activation row behind this thread's B column
    {
        constexpr int G = (BPW + 3) / 4;  // groups of four blocks
#pragma unroll
        for (int gr = 0; gr < G; ++gr) {
            float4 v[4][2];
            int qsum[4] = {0, 0, 0, 0};
            float amax = 0.f;
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                const int j = 4 * gr + jj;
                if (j < BPW && xrow < p.M) {
                    const int k0 = 32 * (warp * BPW + j);
                    v[jj][0] = i8_load_x4(p.X, p.x_dtype, p.K, xrow, k0 + 4 * t);
                    v[jj][1] = i8_load_x4(p.X, p.x_dtype, p.K, xrow, k0 + 16 + 4 * t);
                } else {
                    v[jj][0] = v[jj][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[jj][h].x), fabsf(v[jj][h].y)), fmaxf(fabsf(v[jj][h].z), fabsf(v[jj][h].w))));
            }
            // the four lanes of a quad hold the group's 128 values of row g between them
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            int e = 0;
            if (amax > 0.f && amax < 3.0e38f) e = 13 - (int)((__float_as_uint(amax) >> 23) & 0xFFu) + 127;
            e = max(-126, min(126, e));
            const float s = __uint_as_float((uint32_t)(e + 127) << 23);
            const float inv = __uint_as_float((uint32_t)(127 - e) << 23);
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                const int j = 4 * gr + jj;
                if (j < BPW) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const float f[4] = {v[jj][h].x, v[jj][h].y, v[jj][h].z, v[jj][h].w};
                        uint32_t hi = 0, lo = 0;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int q = max(-16383, min(16383, __float2int_rn(f[i] * s)));
                            hi |= (uint32_t)((q >> 7) & 0xFF) << (8 * i);  // -128 .. 127
                            lo |= (uint32_t)(q & 127) << (8 * i);          // 0 .. 127
                            const int term = PACK ? (g >= 4 ? (q & 127) : (q >> 7)) : q;
                            if (h == 0 && i == 0) qsum[jj] = term;
                            else qsum[jj] += term;
                        }
                        if constexpr (PACK) {
                            xb[j][h] = g >= 4 ? lo : hi;
                        } else {
                            xb[j][h] = hi;
                            xb[j][2 + h] = lo;
                        }
                    }
                }
            }
            if constexpr (FMT == kQ4_K) {
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    const int j = 4 * gr + jj;
                    if (j < BPW) {
                        int sm = qsum[jj];  // the quad's four lanes hold the k-step's 32 values of row g
                        sm += __shfl_xor_sync(0xffffffffu, sm, 1);
                        sm += __shfl_xor_sync(0xffffffffu, sm, 2);
                        xsum[j][0] = __shfl_sync(0xffffffffu, sm, 8 * t);
                        xsum[j][1] = __shfl_sync(0xffffffffu, sm, 8 * t + 4);
                    }
                }
            }
            // the accumulator's columns are 2t and 2t+1: their scales sit in the quads g' = 2t and 2t+1
            cs[gr][0] = __shfl_sync(0xffffffffu, inv, 8 * t);
            cs[gr][1] = __shfl_sync(0xffffffffu, inv, 8 * t + 4);
        }
    }

    bool live = true;
    int stage = 0;
    uint32_t parity = 0;
    for (int i = 0; i < n_tiles; ++i) {
        if (live) {
            const bool ok = wait_or_abort(smem_u32(&bar_full[stage]), parity, &abort_flag, p.status, kDevTimeoutFull, wait_limit);
            live = __all_sync(0xffffffffu, ok);
        }
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        if (live) {
            if constexpr (FMT == kQ8_0) {
                const uint32_t ra0 = sbase + (uint32_t)stage * stage_bytes + (uint32_t)(g * p.row_stride) + (uint32_t)(34 * warp * BPW);
                const uint32_t rb0 = ra0 + 8u * (uint32_t)p.row_stride;
#pragma unroll
                for (int j = 0; j < BPW; ++j) {
                    const uint32_t ra = ra0 + 34u * j + 4u * t, rb = rb0 + 34u * j + 4u * t;
                    uint32_t a[4];
                    // warp * BPW is even, so the block's parity is j's: an even block starts on a word and
                    // its quants two bytes in, an odd block's quants start on a word
                    if ((j & 1) == 0) {
                        a[0] = __funnelshift_r(lds32i<0>(ra), lds32i<4>(ra), 16);
                        a[2] = __funnelshift_r(lds32i<16>(ra), lds32i<20>(ra), 16);
                        a[1] = __funnelshift_r(lds32i<0>(rb), lds32i<4>(rb), 16);
                        a[3] = __funnelshift_r(lds32i<16>(rb), lds32i<20>(rb), 16);
                    } else {
                        a[0] = lds32i<2>(ra);
                        a[2] = lds32i<18>(ra);
                        a[1] = lds32i<2>(rb);
                        a[3] = lds32i<18>(rb);
                    }
                    const float dA = h2f(lds16(ra - 4u * t)), dB = h2f(lds16(rb - 4u * t));
                    int ch[4] = {0, 0, 0, 0};
                    mma_s8(ch, a, xb[j][0], xb[j][1]);
                    if constexpr (!PACK) {
                        int cl[4] = {0, 0, 0, 0};
                        mma_s8(cl, a, xb[j][2], xb[j][3]);
#pragma unroll
                        for (int i = 0; i < 4; ++i) ch[i] = ch[i] * 128 + cl[i];
                    }
                    const float s0 = cs[j >> 2][0], s1 = cs[j >> 2][1];
                    acc[0] = fmaf((float)ch[0], dA * s0, acc[0]);
                    acc[1] = fmaf((float)ch[1], dA * s1, acc[1]);
                    acc[2] = fmaf((float)ch[2], dB * s0, acc[2]);
                    acc[3] = fmaf((float)ch[3], dB * s1, acc[3]);
                }
            } else {
                // this warp's sub-blocks are s0 .. s0 + BPW - 1 of block `blk` of every row (s0 = 0 or 4)
                const int sb0 = warp * BPW, blk = sb0 >> 3, s0 = sb0 & 7;
                const uint32_t ba = sbase + (uint32_t)stage * stage_bytes + (uint32_t)(g * p.row_stride) + 144u * (uint32_t)blk;
                const uint32_t bb = ba + 8u * (uint32_t)p.row_stride;
                const uint4 hA = lds128i<0>(ba), hB = lds128i<0>(bb);
                // the six-bit scales / mins of the warp's sub-blocks, one per byte (sub-blocks 0-3: low words, 4-7: high)
                const bool upper = s0 >= 4;
                uint32_t scw[2][2], mw[2][2];  // [row][word of four sub-blocks]
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const uint4 h = r ? hB : hA;
                    const uint32_t sclo = h.y & 0x3f3f3f3fu, schi = (h.w & 0x0f0f0f0fu) | ((h.y >> 2) & 0x30303030u);
                    const uint32_t mlo = h.z & 0x3f3f3f3fu, mhi = ((h.w >> 4) & 0x0f0f0f0fu) | ((h.z >> 2) & 0x30303030u);
                    scw[r][0] = upper ? schi : sclo;
                    mw[r][0] = upper ? mhi : mlo;
                    scw[r][1] = schi;  // only BPW = 8 reaches the second word
                    mw[r][1] = mhi;
                }
                const float dA = h2f(hA.x & 0xFFFFu), dmA = h2f(hA.x >> 16), dB = h2f(hB.x & 0xFFFFu), dmB = h2f(hB.x >> 16);
#pragma unroll
                for (int gr = 0; gr < BPW / 4; ++gr) {
                    int i1[4] = {0, 0, 0, 0}, i2[4] = {0, 0, 0, 0};
                    uint32_t wA0 = 0, wA1 = 0, wB0 = 0, wB1 = 0;
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        const int j = 4 * gr + jj;
                        if ((jj & 1) == 0) {  // a pair of sub-blocks shares its 32 bytes of quants
                            const uint32_t qo = 16u + 32u * (uint32_t)((s0 + j) >> 1) + 4u * t;
                            wA0 = lds32i<0>(ba + qo); wA1 = lds32i<16>(ba + qo);
                            wB0 = lds32i<0>(bb + qo); wB1 = lds32i<16>(bb + qo);
                        }
                        const uint32_t sh = (jj & 1) ? 4u : 0u;
                        const uint32_t a[4] = {(wA0 >> sh) & 0x0F0F0F0Fu, (wB0 >> sh) & 0x0F0F0F0Fu, (wA1 >> sh) & 0x0F0F0F0Fu, (wB1 >> sh) & 0x0F0F0F0Fu};
                        int ch[4] = {0, 0, 0, 0};
                        mma_s8(ch, a, xb[j][0], xb[j][1]);
                        if constexpr (!PACK) {
                            int cl[4] = {0, 0, 0, 0};
                            mma_s8(cl, a, xb[j][2], xb[j][3]);
#pragma unroll
                            for (int i = 0; i < 4; ++i) ch[i] = ch[i] * 128 + cl[i];
                        }
                        const int scA = (int)((scw[0][gr] >> (8 * jj)) & 0xFFu), scB = (int)((scw[1][gr] >> (8 * jj)) & 0xFFu);
                        const int mA = (int)((mw[0][gr] >> (8 * jj)) & 0xFFu), mB = (int)((mw[1][gr] >> (8 * jj)) & 0xFFu);
                        // |sc * dot| <= 63 * 32 * 15 * 16383 = 4.95e8: four of them fit an int32
                        i1[0] += scA * ch[0];
                        i1[1] += scA * ch[1];
                        i1[2] += scB * ch[2];
                        i1[3] += scB * ch[3];
                        i2[0] += mA * xsum[j][0];
                        i2[1] += mA * xsum[j][1];
                        i2[2] += mB * xsum[j][0];
                        i2[3] += mB * xsum[j][1];
                    }
                    acc[0] = fmaf(cs[gr][0], dA * (float)i1[0] - dmA * (float)i2[0], acc[0]);
                    acc[1] = fmaf(cs[gr][1], dA * (float)i1[1] - dmA * (float)i2[1], acc[1]);
                    acc[2] = fmaf(cs[gr][0], dB * (float)i1[2] - dmB * (float)i2[2], acc[2]);
                    acc[3] = fmaf(cs[gr][1], dB * (float)i1[3] - dmB * (float)i2[3], acc[3]);
                }
            }
        }
        // ---- the warps' partial sums meet in shared memory (two buffers, alternating by tile)
        const uint32_t part = part_base + (uint32_t)(i & 1) * (kI8Warps * 128 * 4);
        sts32(part + (uint32_t)((warp * 128 + g * 8 + 2 * t) * 4), __float_as_uint(acc[0]));
        sts32(part + (uint32_t)((warp * 128 + g * 8 + 2 * t + 1) * 4), __float_as_uint(acc[1]));
        sts32(part + (uint32_t)((warp * 128 + (g + 8) * 8 + 2 * t) * 4), __float_as_uint(acc[2]));
        sts32(part + (uint32_t)((warp * 128 + (g + 8) * 8 + 2 * t + 1) * 4), __float_as_uint(acc[3]));
        __syncthreads();  // every warp is done with the stage and has left its partial sums
        if (lane == 0 && live && i + p.n_stages < n_tiles) feed(i + p.n_stages, stage);
        if (tid < 128 && live && !*(volatile int*)&abort_flag) {
            const int r = tid >> 3, m = tid & 7, n = kI8TileRows * (tile_first + i) + r;
            if (m < p.M && n < p.N && (!PACK || m < 4)) {
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < kI8Warps; ++w) s += __uint_as_float(lds32i<0>(part + (uint32_t)((w * 128 + tid) * 4)));  // fixed order
                if constexpr (PACK) {  // column m is the hi plane, column m + 4 the lo plane
                    float sl = 0.f;
#pragma unroll
                    for (int w = 0; w < kI8Warps; ++w) sl += __uint_as_float(lds32i<16>(part + (uint32_t)((w * 128 + tid) * 4)));
                    s = fmaf(128.0f, s, sl);
                }
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
        if (++stage == p.n_stages) {
            stage = 0;
            parity ^= 1;
        }
    }
}

// ---- host side ------------------------------------------------------------------------

static int g_opt_i8 = 1;
void i8_set_enabled(int v) { g_opt_i8 = v < 0 ? 0 : (v > 2 ? 2 : v); }
int i8_get_enabled() { return g_opt_i8; }
int dp_get_wait_limit_us();

template <int FMT, int BPW, bool PACK>
static int launch_i8(const I8Params& p, int grid, size_t smem, cudaStream_t st) {
    auto kern = gemv_i8_kernel<FMT, BPW, PACK>;
    static bool configured[64] = {};
    int dev = 0;
    B200Q_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        B200Q_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 512));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kI8Warps * 32);
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

// Launches the integer tensor-core kernel when the call qualifies (*taken = true): Q8_0 or Q4_K, two to
// eight activation rows, K = 2048 or 4096, 16-byte aligned weights.
int launch_gemv_i8(int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype, int M, int N, int K,
                   int sms, int* status, cudaStream_t st, bool* taken) {
    *taken = false;
    if (!g_opt_i8 || (fmt != kQ8_0 && fmt != kQ4_K) || M < 2 || M > 8 || (K != 2048 && K != 4096) || N < 1) return B200Q_OK;
    // measured: two rows of Q4_K are faster on the dp2a kernel (11.4 against 12.6 us on 14336 x 4096); option 2 takes them too
    if (g_opt_i8 == 1 && fmt == kQ4_K && M == 2) return B200Q_OK;
    if ((reinterpret_cast<uintptr_t>(W) & 15) != 0) return B200Q_OK;
    if (x_dtype != B200Q_DT_F32 && (reinterpret_cast<uintptr_t>(X) & 7) != 0) return B200Q_OK;
    if (x_dtype == B200Q_DT_F32 && (reinterpret_cast<uintptr_t>(X) & 15) != 0) return B200Q_OK;
    I8Params p = {};
    p.W = static_cast<const uint8_t*>(W);
    p.X = X;
    p.bias = bias;
    p.Y = Y;
    p.status = status;
    p.M = M;
    p.N = N;
    p.K = K;
    p.x_dtype = x_dtype;
    p.y_dtype = y_dtype;
    p.row_bytes = fmt == kQ8_0 ? (K / 32) * 34 : (K / 256) * 144;
    p.row_stride = p.row_bytes + 16;  // a multiple of 32 words + 4: the eight rows of a fragment load fall into different banks
    const int tiles = (N + kI8TileRows - 1) / kI8TileRows;
    int grid = stream_get_option(3) > 0 ? stream_get_option(3) : sms;
    if (grid > tiles) grid = tiles;
    p.tile_q = tiles / grid;
    p.tile_r = tiles % grid;
    const int most = p.tile_q + (p.tile_r ? 1 : 0);
    const size_t stage = (size_t)kI8TileRows * p.row_stride, fixed = 128 + 2 * kI8Warps * 128 * sizeof(float);
    const int fit = (int)((227 * 1024 - 512 - fixed) / stage);  // three stages of Q8_0 at K = 4096, five of Q4_K
    p.n_stages = most < kI8MaxStages ? most : kI8MaxStages;
    if (p.n_stages > fit) p.n_stages = fit;
    if (p.n_stages < 1) return B200Q_OK;
    p.wait_limit_us = (unsigned int)dp_get_wait_limit_us();
    const size_t smem = fixed + (size_t)p.n_stages * stage;
    int rc;
    if (M <= 4)
        rc = fmt == kQ8_0 ? (K == 4096 ? launch_i8<kQ8_0, 8, true>(p, grid, smem, st) : launch_i8<kQ8_0, 4, true>(p, grid, smem, st))
                          : (K == 4096 ? launch_i8<kQ4_K, 8, true>(p, grid, smem, st) : launch_i8<kQ4_K, 4, true>(p, grid, smem, st));
    else
        rc = fmt == kQ8_0 ? (K == 4096 ? launch_i8<kQ8_0, 8, false>(p, grid, smem, st) : launch_i8<kQ8_0, 4, false>(p, grid, smem, st))
                          : (K == 4096 ? launch_i8<kQ4_K, 8, false>(p, grid, smem, st) : launch_i8<kQ4_K, 4, false>(p, grid, smem, st));
    if (rc) return rc;
    *taken = true;
    return B200Q_OK;
}

}  // namespace b200q

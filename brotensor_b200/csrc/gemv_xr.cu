// Decode GEMV for one activation row and rows of at most 4096 elements, Q4_K and Q6_K (sm_100a): the
// activation-resident form of the integer-dot-product GEMV of gemv_dp.cu.
//
// What is different from gemv_dp.cu, and why:
//   * A lane's 128-element activation group is the same for every weight row when a row has at most
//     32 groups, so the lane loads it ONCE per launch and keeps it in registers (64 registers of
//     int16 pairs, plus the four sub-block sums and the group's scale). In gemv_dp.cu the activations
//     are re-read from shared memory for every row pair: 16 of an item's 28 128-bit loads.
//   * The ring's unit is one ROW PAIR (one bulk copy, one barrier per slot), and every warp feeds
//     itself: it owns three slots, and its first lane issues the copy of the pair that will use a slot
//     next the moment the warp is done with the slot. There is no producer warp, no "empty" barrier,
//     no hand-over between warps, and a slot meets one warp only, in order.
//   * A CTA's rows are split in pairs over all SMs, not in 16-row tiles over a tile-balanced grid:
//     14336 rows are 48.4 pairs per SM (three pairs per warp and one more for one warp), where the
//     tile form runs 7 tiles on 128 of the 148 SMs (four rounds on one of its two pipelines).
//   * The ring is filled in steps (first slot of every warp at entry, second once the activation loads
//     are on their way, third once the activations are staged): copies in flight share an SM's ingest
//     rate, so a ring filled in one burst delivers its first bytes as late as its last and delays the
//     activation loads queued behind it (measured: first item 4.5 instead of 2.7 us after entry).
//
// One CTA of 16 warps per SM, 128 registers per thread (the whole register file: the activations
// are replicated in every warp). Measured on B200 against gemv_dp.cu (back-to-back launches under
// programmatic dependent launch, weights rotating through more than the L2): 14336 x 4096 6.7 vs
// 7.4-7.6 us, 28672 x 4096 10.8 vs 12.6, 1024 x 4096 2.2 vs 2.4; between about 4096 and 8192 rows it
// is 0.1-0.4 us slower (one round of items that all wait for the same burst), which is why the
// dispatcher sends those to gemv_dp.cu.
// A variant sized for two CTAs per SM (7 or 8 warps, half the shared memory), so that the next launch
// of the stream could move in beside the running one and prefetch, was measured too: it is slower
// (7.6-8.5 us) - half of the SM's warps sit parked in griddepcontrol.wait, and the items are bound
// by instruction issue, not by memory. Giving the one pair that a CTA with 16 n + 1 pairs ends on (14336 rows:
// 48 or 49 pairs per CTA; the 49th costs one warp 0.54 us while fifteen wait) to two warps, a row each, was
// measured as well: 6.87 against 6.74 us - the bookkeeping in every item costs more than the shorter tail saves.
//
// Q6_K (K = 2048 or 4096) runs through the same kernel with the half-group work unit of gemv_dp.cu: a lane
// keeps the 64 activations of its half group of each 2048-element slice, their 16-element sums and the
// group scales; a row pair is 6720 bytes, so a warp has two ring slots instead of three. The gain is
// smaller than for Q4_K (the 6-bit unpack, not the activation loads, is most of a Q6_K item):
// 16032 x 4096 11.2 against 11.6 us, 32064 x 4096 18.5 against 19.7; below 8192 rows it loses.
//
// Arithmetic is exactly gemv_dp.cu's (same staging of the activations, same integer dot products,
// same FP32 combination per group, same butterfly over the lanes), so results are bit-identical to it.
//
// Takes the place of brotensor's linear_q4k_fp16_gemv_kernel (src/cuda/q4k.cu:159-224) and
// linear_q6k_fp16_gemv_kernel (src/cuda/q6k.cu:117-176).
#include "dp_common.cuh"

namespace b200q {

constexpr int kXrMaxSlots = 48;
constexpr int kXrMaxK = 4096;

struct XrParams {
    const uint8_t* W;
    const void* X;
    const void* bias;
    void* Y;
    int* status;
    int N, K;
    int x_dtype, y_dtype;
    int row_bytes;
    int n_slots;         // ring depth in row pairs
    int pair_q, pair_r;  // CTA b owns pair_q + (b < pair_r) row pairs, starting at b * pair_q + min(b, pair_r)
    unsigned int wait_limit_us;
#ifdef B200Q_TRACE
    unsigned long long* trace;
#endif
};

// shared-memory layout (bytes from the 128-byte aligned base)
constexpr uint32_t kXrOffX = 0;                                 // 32 groups x 272 bytes of int16 activations
constexpr uint32_t kXrOffScale = 32 * kXGroupStride;            // 32 floats: 2^-e per group
constexpr uint32_t kXrOffSums = kXrOffScale + 128;              // Q4_K: 128 sums over 32 elements; Q6_K: 256 sums over 16
constexpr uint32_t kXrOffRing = kXrOffSums + 1024;              // n_slots x 2 rows
constexpr size_t kXrFixedSmem = kXrOffRing + 128;               // plus alignment slack

// Stages segment `idx` (eight activations) of the row: int16 with the group's power-of-two scale,
// as x_store_seg of gemv_dp.cu does for one activation row. Called by whole warps.
template <int FMT>
__device__ __forceinline__ void xr_stage_seg(uint32_t sbase, int idx, const float (&v)[8]) {
    const int gg = idx >> 4, i = idx & 15;
    float amax = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(v[k]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 8));
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
    sts128(sbase + kXrOffX + (uint32_t)(gg * kXGroupStride + (i << 4)), o);
    if (i == 0) sts32(sbase + kXrOffScale + (uint32_t)gg * 4, (uint32_t)(127 - e) << 23);
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    if constexpr (FMT == kQ6_K) {  // sums over 16 elements = 2 segments
        if ((i & 1) == 0) sts32(sbase + kXrOffSums + (uint32_t)(idx >> 1) * 4, (uint32_t)sum);
    } else {                        // sums over 32 elements = 4 segments
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if ((i & 3) == 0) sts32(sbase + kXrOffSums + (uint32_t)(idx >> 2) * 4, (uint32_t)sum);
    }
}

// q4k_dot of dp_common.cuh against activations x[OFF .. OFF + 7] of the resident group (constant
// indices only, so that the group stays in registers).
template <int OFF>
__device__ __forceinline__ void xr_dot(const uint4& q0, const uint4& q1, const uint4 (&x)[16], int& cl, int& ch) {
    const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    int a0 = 0, a1 = 0, b0 = 0, b1 = 0;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        const uint32_t l0 = w[2 * s] & 0x0F0F0F0Fu, l1 = w[2 * s + 1] & 0x0F0F0F0Fu;
        const uint32_t h0 = w[2 * s] & 0xF0F0F0F0u, h1 = w[2 * s + 1] & 0xF0F0F0F0u;
        a0 = dp2a_lo_su(x[OFF + s].x, l0, a0);
        a0 = dp2a_hi_su(x[OFF + s].y, l0, a0);
        a1 = dp2a_lo_su(x[OFF + s].z, l1, a1);
        a1 = dp2a_hi_su(x[OFF + s].w, l1, a1);
        b0 = dp2a_lo_su(x[OFF + 4 + s].x, h0, b0);
        b0 = dp2a_hi_su(x[OFF + 4 + s].y, h0, b0);
        b1 = dp2a_lo_su(x[OFF + 4 + s].z, h1, b1);
        b1 = dp2a_hi_su(x[OFF + 4 + s].w, h1, b1);
    }
    cl = a0 + a1;
    ch = (b0 + b1) >> 4;  // exact: every term is a multiple of 16
}

// One row (the lane's half block of it) against the lane's resident activations.
__device__ __forceinline__ float xr_row(uint32_t pr, int hb, const uint4 (&x)[16], const uint4& sv, float xs) {
    const uint32_t qa = pr + 64u * hb;
    const uint4 h = lds128i<0>(pr);
    const uint4 q0 = lds128i<16>(qa), q1 = lds128i<32>(qa), q2 = lds128i<48>(qa), q3 = lds128i<64>(qa);
    const uint32_t sclo = h.y & 0x3f3f3f3fu, schi = (h.w & 0x0f0f0f0fu) | ((h.y >> 2) & 0x30303030u);
    const uint32_t mlo = h.z & 0x3f3f3f3fu, mhi = ((h.w >> 4) & 0x0f0f0f0fu) | ((h.z >> 2) & 0x30303030u);
    const uint32_t scw = hb ? schi : sclo, mw = hb ? mhi : mlo;
    const float d = h2f(h.x & 0xFFFFu), dm = h2f(h.x >> 16);
    int cl, ch;
    xr_dot<0>(q0, q1, x, cl, ch);
    int isum = (int)(scw & 0xFFu) * cl + (int)((scw >> 8) & 0xFFu) * ch;
    xr_dot<8>(q2, q3, x, cl, ch);
    isum += (int)((scw >> 16) & 0xFFu) * cl + (int)(scw >> 24) * ch;
    const int imin = (int)(mw & 0xFFu) * (int)sv.x + (int)((mw >> 8) & 0xFFu) * (int)sv.y + (int)((mw >> 16) & 0xFFu) * (int)sv.z +
                     (int)(mw >> 24) * (int)sv.w;
    return xs * (d * (float)isum - dm * (float)imin);
}

// ---- Q6_K: one row's half group (64 elements: {32 Q + 16 H + i}, Q = 0..3, i = 0..15, of group gi) against
// the lane's resident activations x[2 Q], x[2 Q + 1] and their 16-element sums sx[Q]; the arithmetic of
// item_q6k_half / q6_sub_h in gemv_dp.cu. Returns d * sum_Q sc_Q * (dot_Q - 32 * sx_Q).
__device__ __forceinline__ uint32_t xr_lds32(uint32_t a) { return lds32i<0>(a); }
__device__ __forceinline__ float xr_q6k_row(uint32_t row, int gi, int H, const uint4 (&x)[8], const int (&sx)[4], float& d_out) {
    const int bi = gi >> 1, G = gi & 1;
    const uint32_t sh = (uint32_t)(bi & 1) * 16u;  // odd blocks start at 2 (mod 4): aligned words + funnel shift
    const uint32_t L = row + (uint32_t)(bi * 210 - (bi & 1) * 2);
    const uint32_t La = L + 64u * G + 16u * H, Lh = L + 128u + 32u * G + 16u * H, Ls = L + 192u + 8u * G;
    uint32_t ql[8], qh[4], su[2];
    {
        uint32_t ra[5], rb[5], rh[5], rs[3];
#pragma unroll
        for (int k = 0; k < 5; ++k) {
            ra[k] = xr_lds32(La + 4u * k);
            rb[k] = xr_lds32(La + 32u + 4u * k);
            rh[k] = xr_lds32(Lh + 4u * k);
        }
#pragma unroll
        for (int k = 0; k < 3; ++k) rs[k] = xr_lds32(Ls + 4u * k);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            ql[k] = __funnelshift_r(ra[k], ra[k + 1], sh);
            ql[4 + k] = __funnelshift_r(rb[k], rb[k + 1], sh);
            qh[k] = __funnelshift_r(rh[k], rh[k + 1], sh);
        }
        su[0] = __funnelshift_r(rs[0], rs[1], sh) ^ 0x80808080u;
        su[1] = __funnelshift_r(rs[1], rs[2], sh) ^ 0x80808080u;
    }
    d_out = h2f((lds32i<208>(L) >> sh) & 0xFFFFu);
    float accg = 0.f;
#pragma unroll
    for (int Q = 0; Q < 4; ++Q) {
        uint32_t v[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const uint32_t a = ql[4 * (Q & 1) + w], hb = qh[w];
            const uint32_t nib = (Q < 2 ? a : (a >> 4)) & 0x0F0F0F0Fu;
            const uint32_t h2 = (Q == 0 ? hb << 4 : Q == 1 ? hb << 2 : Q == 2 ? hb : hb >> 2) & 0x30303030u;
            v[w] = nib | h2;
        }
        // int8 scale byte 2 (Q & 1) + H of the word (bytes xor-ed with 0x80) -> exact float
        const float scf = __uint_as_float(__byte_perm(su[Q >> 1], 0x4B000000u, 0x7440 | (2 * (Q & 1) + H))) - 8388736.0f;
        const uint4 x0 = x[2 * Q], x1 = x[2 * Q + 1];
        int c0 = 0, c1 = 0;
        c0 = dp2a_lo_su(x0.x, v[0], c0);
        c0 = dp2a_hi_su(x0.y, v[0], c0);
        c1 = dp2a_lo_su(x0.z, v[1], c1);
        c1 = dp2a_hi_su(x0.w, v[1], c1);
        c0 = dp2a_lo_su(x1.x, v[2], c0);
        c0 = dp2a_hi_su(x1.y, v[2], c0);
        c1 = dp2a_lo_su(x1.z, v[3], c1);
        c1 = dp2a_hi_su(x1.w, v[3], c1);
        accg = fmaf(scf, (float)(c0 + c1 - 32 * sx[Q]), accg);
    }
    return accg;
}

template <int FMT, int CW>
__global__ void __launch_bounds__(CW * 32, 1) gemv_xr_kernel(const __grid_constant__ XrParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 127u) & ~127u;
    __shared__ uint64_t bar_full[kXrMaxSlots];
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = (int)blockIdx.x;
    const int pair_first = cta * p.pair_q + min(cta, p.pair_r), n_items = p.pair_q + (cta < p.pair_r ? 1 : 0);
    const uint32_t slot_bytes = 2u * (uint32_t)p.row_bytes;
    const uint32_t ring = sbase + kXrOffRing;
    const uint64_t wait_limit = p.wait_limit_us ? (uint64_t)p.wait_limit_us * 1000ull : kWaitLimitNs;
    TRACE_STAMP(tid == 0, 0);

    // Every warp feeds itself: its items are warp, warp + CW, ..., its ring slots warp, warp + CW, ...
    // (n_slots is a multiple of CW), and its first lane issues the copy of the item that will use a slot
    // next as soon as the warp is done with the slot. No producer warp, no "empty" barriers, and a slot
    // meets one warp only, in order, so a barrier's two parities cannot be mistaken for one another.
    // Weights do not depend on the stream-ordered predecessor: the first copies go out before
    // griddepcontrol.wait.
    if (tid == 0) abort_flag = 0;
    // The copy of item `it` into its slot; called by a warp's first lane.
    auto feed = [&](int it, int s) {
        if (it >= n_items || s >= p.n_slots) return;
        const int row = 2 * (pair_first + it);
        const uint32_t bytes = (uint32_t)min(2, p.N - row) * (uint32_t)p.row_bytes;
        const uint32_t full = smem_u32(&bar_full[s]);
        mbar_arrive_expect_tx(full, bytes);
        bulk_g2s(ring + (uint32_t)s * slot_bytes, p.W + (size_t)row * p.row_bytes, bytes, full);
    };
    // A deep ring filled in one burst delivers its first bytes as late as its last (the copies in
    // flight share the SM's ingest rate), and loads issued behind the burst wait for it. So the ring is
    // filled in steps: each warp's first slot now, its second once the activation loads are on their
    // way, its third once the activations are staged.
    if (lane == 0) {
        for (int s = warp; s < p.n_slots; s += CW) mbar_init(smem_u32(&bar_full[s]), 1);
        fence_mbar_init();
        feed(warp, warp);
    }
    TRACE_STAMP(tid == 0, 7);
    grid_dep_launch();
    TRACE_STAMP(tid == 0, 1);

    // ---- consumers
    grid_dep_wait();  // activations (and Y) belong to the stream-ordered predecessor
    TRACE_STAMP(tid == 0, 2);
    {
        // K % 256 == 0 and CW * 32 % 32 == 0: whole warps are in or out. All of a thread's loads go out
        // before the first is converted (one load latency, not one per segment): the loads are
        // unconditional (a segment past the row's end re-reads the last one) and the element type is
        // switched once around them, so that nothing separates them.
        constexpr int U = (kXrMaxK / 8 + CW * 32 - 1) / (CW * 32);
        const int segs = p.K >> 3;
        float v[U][8];
        if (p.x_dtype == B200Q_DT_F32) {
            float4 r[U][2];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const float4* X = reinterpret_cast<const float4*>(p.X) + 2 * min(tid + u * CW * 32, segs - 1);
                r[u][0] = __ldg(X);
                r[u][1] = __ldg(X + 1);
            }
            if (lane == 0) feed(warp + CW, warp + CW);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                v[u][0] = r[u][0].x; v[u][1] = r[u][0].y; v[u][2] = r[u][0].z; v[u][3] = r[u][0].w;
                v[u][4] = r[u][1].x; v[u][5] = r[u][1].y; v[u][6] = r[u][1].z; v[u][7] = r[u][1].w;
            }
        } else {
            uint4 r[U];
#pragma unroll
            for (int u = 0; u < U; ++u) r[u] = __ldg(reinterpret_cast<const uint4*>(p.X) + min(tid + u * CW * 32, segs - 1));
            if (lane == 0) feed(warp + CW, warp + CW);
#pragma unroll
            for (int u = 0; u < U; ++u) {
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
        for (int u = 0; u < U; ++u)
            if (tid + u * CW * 32 < segs) xr_stage_seg<FMT>(sbase, tid + u * CW * 32, v[u]);
    }
    if (lane == 0) feed(warp + 2 * CW, warp + 2 * CW);
    asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
    // the lane's activations, resident from here on.
    // Q4_K: its 128-element group (lanes past the row's last group work on zeros).
    // Q6_K: the half group (lane % 16, lane / 16) of the row's first 2048 elements in x[0..7] and of the
    // second 2048 (K = 4096) in x[8..15], with their 16-element sums and group scales.
    const bool active = FMT == kQ6_K ? true : lane < (p.K >> 7);
    uint4 x[16];
    uint4 sv = make_uint4(0u, 0u, 0u, 0u);
    float xs = 0.f;
    int sx6[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
    float xs6[2] = {0.f, 0.f};
    const int H6 = lane >> 4, g6 = lane & 15;
    const bool two = p.K > 2048;  // Q6_K: a second slice
    if constexpr (FMT == kQ6_K) {
#pragma unroll
        for (int sl = 0; sl < 2; ++sl) {
            const int gg = (sl && two) ? 16 + g6 : g6;  // without a second slice the loads repeat the first (scale 0)
            const uint32_t xg = sbase + kXrOffX + (uint32_t)(gg * kXGroupStride + 32 * H6);
            x[8 * sl + 0] = lds128i<0>(xg);   x[8 * sl + 1] = lds128i<16>(xg);
            x[8 * sl + 2] = lds128i<64>(xg);  x[8 * sl + 3] = lds128i<80>(xg);
            x[8 * sl + 4] = lds128i<128>(xg); x[8 * sl + 5] = lds128i<144>(xg);
            x[8 * sl + 6] = lds128i<192>(xg); x[8 * sl + 7] = lds128i<208>(xg);
            if (sl == 0 || two) {
#pragma unroll
                for (int Q = 0; Q < 4; ++Q) sx6[sl][Q] = (int)lds32i<0>(sbase + kXrOffSums + (uint32_t)((8 * gg + 2 * Q + H6) * 4));
                xs6[sl] = __uint_as_float(lds32i<0>(sbase + kXrOffScale + (uint32_t)gg * 4u));
            }
        }
    } else {
        const uint32_t xg = sbase + kXrOffX + (uint32_t)((active ? lane : 0) * kXGroupStride);
        x[0] = lds128i<0>(xg); x[1] = lds128i<16>(xg); x[2] = lds128i<32>(xg); x[3] = lds128i<48>(xg);
        x[4] = lds128i<64>(xg); x[5] = lds128i<80>(xg); x[6] = lds128i<96>(xg); x[7] = lds128i<112>(xg);
        x[8] = lds128i<128>(xg); x[9] = lds128i<144>(xg); x[10] = lds128i<160>(xg); x[11] = lds128i<176>(xg);
        x[12] = lds128i<192>(xg); x[13] = lds128i<208>(xg); x[14] = lds128i<224>(xg); x[15] = lds128i<240>(xg);
        if (active) {
            sv = lds128i<0>(sbase + kXrOffSums + (uint32_t)lane * 16u);
            xs = __uint_as_float(lds32i<0>(sbase + kXrOffScale + (uint32_t)lane * 4u));
        }
    }
    TRACE_STAMP(tid == 0, 3);

    // the lane's half block inside a row: block lane / 2, half lane % 2 (inactive lanes read block 0, scale 0)
    const uint32_t lane_off = FMT == kQ6_K ? 0u : (active ? (uint32_t)(lane >> 1) * 144u : 0u);
    const int hb = lane & 1;
    bool live = true;
    // Deferred reduction: the lanes' partial sums of up to four items (eight rows) are kept and
    // reduced together - nine shuffles for eight rows - in the butterfly order of gemv_dp.cu.
    float hold[3][2] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};  // the three items before the current one, newest first
    int held = 0;
    // this warp's items are warp, warp + CW, ...; their slots are warp, warp + CW, ... (mod n_slots)
    int slot = warp;
    uint32_t parity = 0;
    for (int i = warp; i < n_items; i += CW) {
        if (live) {
            const bool ok = wait_or_abort(smem_u32(&bar_full[slot]), parity, &abort_flag, p.status, kDevTimeoutFull, wait_limit);
            live = __all_sync(0xffffffffu, ok);
        }
        TRACE_STAMP(tid == 0 && i == 0, 4);
        float a0 = 0.f, a1 = 0.f;
        if (live) {
            const int row = 2 * (pair_first + i);
            const uint32_t prA = ring + (uint32_t)slot * slot_bytes + lane_off;
            const uint32_t prB = (row + 1 < p.N) ? prA + (uint32_t)p.row_bytes : prA;  // odd row count: the sum is dropped
            if constexpr (FMT == kQ6_K) {
                const uint32_t rA = prA - lane_off, rB = prB - lane_off;  // row bases
                const uint4(&xa)[8] = *reinterpret_cast<const uint4(*)[8]>(&x[0]);
                const uint4(&xb)[8] = *reinterpret_cast<const uint4(*)[8]>(&x[8]);
                float d;
                float g0 = xr_q6k_row(rA, g6, H6, xa, sx6[0], d);
                a0 = fmaf(d * xs6[0], g0, 0.f);
                g0 = xr_q6k_row(rB, g6, H6, xa, sx6[0], d);
                a1 = fmaf(d * xs6[0], g0, 0.f);
                if (two) {
                    g0 = xr_q6k_row(rA, 16 + g6, H6, xb, sx6[1], d);
                    a0 = fmaf(d * xs6[1], g0, a0);
                    g0 = xr_q6k_row(rB, 16 + g6, H6, xb, sx6[1], d);
                    a1 = fmaf(d * xs6[1], g0, a1);
                }
            } else {
                a0 = xr_row(prA, hb, x, sv, xs);
                a1 = xr_row(prB, hb, x, sv, xs);
            }
            // the slot's bytes are in registers (the sums above depend on every load): refill it
            asm volatile("" ::"f"(a0), "f"(a1) : "memory");
            __syncwarp();
            const int nxt = i + p.n_slots;
            if (lane == 0 && nxt < n_items) {
                const int nrow = 2 * (pair_first + nxt);
                const uint32_t bytes = (uint32_t)min(2, p.N - nrow) * (uint32_t)p.row_bytes;
                const uint32_t full = smem_u32(&bar_full[slot]);
                mbar_arrive_expect_tx(full, bytes);
                bulk_g2s(ring + (uint32_t)slot * slot_bytes, p.W + (size_t)nrow * p.row_bytes, bytes, full);
            }
        }
        TRACE_STAMP(tid == 0 && i / CW < 7, 9 + i / CW);  // warp 0: end of its k-th item
        slot += CW;
        if (slot >= p.n_slots) {
            slot -= p.n_slots;  // n_slots is a multiple of CW: back to this warp's first slot
            parity ^= 1;
        }
        if (++held < 4 && i + CW < n_items) {
            hold[2][0] = hold[1][0]; hold[2][1] = hold[1][1];
            hold[1][0] = hold[0][0]; hold[1][1] = hold[0][1];
            hold[0][0] = a0; hold[0][1] = a1;
            continue;
        }
        const float v[8] = {hold[2][0], hold[2][1], hold[1][0], hold[1][1], hold[0][0], hold[0][1], a0, a1};
        const bool h16 = (lane & 16) != 0, h8 = (lane & 8) != 0, h4 = (lane & 4) != 0;
        float w4[4], w2[2];
#pragma unroll
        for (int k = 0; k < 4; ++k) w4[k] = (h16 ? v[4 + k] : v[k]) + __shfl_xor_sync(0xffffffffu, h16 ? v[k] : v[4 + k], 16);
#pragma unroll
        for (int k = 0; k < 2; ++k) w2[k] = (h8 ? w4[2 + k] : w4[k]) + __shfl_xor_sync(0xffffffffu, h8 ? w4[k] : w4[2 + k], 8);
        float s = (h4 ? w2[1] : w2[0]) + __shfl_xor_sync(0xffffffffu, h4 ? w2[0] : w2[1], 4);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        const int o = (h16 ? 4 : 0) + (h8 ? 2 : 0) + (h4 ? 1 : 0), age = 3 - (o >> 1);  // items ago; row of the pair: o & 1
        if ((lane & 3) == 0 && age < held && live && !*(volatile int*)&abort_flag) {
            const int n = 2 * (pair_first + i - CW * age) + (o & 1);
            if (n < p.N) {
                if (p.bias) {
                    if (p.x_dtype == B200Q_DT_F32) s += static_cast<const float*>(p.bias)[n];
                    else if (p.x_dtype == B200Q_DT_F16) s += __half2float(static_cast<const __half*>(p.bias)[n]);
                    else s += __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[n]);
                }
                if (p.y_dtype == B200Q_DT_F32) static_cast<float*>(p.Y)[n] = s;
                else if (p.y_dtype == B200Q_DT_F16) static_cast<__half*>(p.Y)[n] = __float2half_rn(s);
                else static_cast<__nv_bfloat16*>(p.Y)[n] = __float2bfloat16_rn(s);
            }
        }
        held = 0;
        hold[0][0] = hold[0][1] = hold[1][0] = hold[1][1] = hold[2][0] = hold[2][1] = 0.f;
    }
    TRACE_STAMP(lane == 0, 5);
}

// ---- host side ------------------------------------------------------------------------

// 1: launches that qualify take this kernel; 2: also those in the row range where gemv_dp.cu is faster; 0: off
static int g_opt_xr = 1;
void xr_set_enabled(int v) { g_opt_xr = v < 0 ? 0 : (v > 2 ? 2 : v); }
int xr_get_enabled() { return g_opt_xr; }
int dp_get_wait_limit_us();

// Launches the activation-resident kernel when the call qualifies (*taken = true): Q4_K (K a multiple of
// 256, at most 4096) or Q6_K (K = 2048 or 4096), one activation row, 16-byte aligned weights.
template <int FMT, int CW>
static int launch_gemv_xr_cw(int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype, int M, int N, int K,
                   int sms, int* status, cudaStream_t st, bool* taken) {
    *taken = false;
    if (!g_opt_xr || fmt != FMT || M != 1 || K % 256 != 0 || K > kXrMaxK || K < 256 || N < 1) return B200Q_OK;
    if (FMT == kQ6_K && K != 2048 && K != 4096) return B200Q_OK;  // whole slices of 2048 elements
    // measured crossovers (see the head of this file); very long Q4_K streams run a few percent faster in gemv_dp.cu
    if (g_opt_xr == 1 && FMT == kQ4_K && ((N > 3072 && N < 10240) || N > 65536)) return B200Q_OK;
    if (g_opt_xr == 1 && FMT == kQ6_K && N < 8192) return B200Q_OK;
    if ((reinterpret_cast<uintptr_t>(W) & 15) != 0) return B200Q_OK;
    XrParams p = {};
    p.W = static_cast<const uint8_t*>(W);
    p.X = X;
    p.bias = bias;
    p.Y = Y;
    p.status = status;
    p.N = N;
    p.K = K;
    p.x_dtype = x_dtype;
    p.y_dtype = y_dtype;
    p.row_bytes = (K / 256) * (FMT == kQ6_K ? 210 : 144);
    const int pairs = (N + 1) / 2;
    int grid = stream_get_option(3) > 0 ? stream_get_option(3) : sms;
    if (grid > pairs) grid = pairs;
    p.pair_q = pairs / grid;
    p.pair_r = pairs % grid;
    constexpr size_t kSmemMax = 227 * 1024 - 512;  // all of an SM's shared memory, less this kernel's static part
    const size_t slot = 2 * (size_t)p.row_bytes;
    int slots = (int)((kSmemMax - kXrFixedSmem) / slot);
    if (slots > 3 * CW) slots = 3 * CW;  // three slots per warp: two in flight while one is read
    if (slots > kXrMaxSlots) slots = kXrMaxSlots;
    const int most = p.pair_q + (p.pair_r ? 1 : 0);
    // a ring deeper than the CTA's items only takes shared memory from its neighbour; a whole number of
    // slots per consumer warp, so that a slot always meets the same warp
    const int need = ((most + CW - 1) / CW) * CW;
    if (slots > need) slots = need;
    slots -= slots % CW;
    if (slots < CW) return B200Q_OK;
    p.n_slots = slots;
    p.wait_limit_us = (unsigned int)dp_get_wait_limit_us();
#ifdef B200Q_TRACE
    p.trace = dp_trace_next(grid);
#endif
    const size_t smem = kXrFixedSmem + (size_t)slots * slot;
    auto kern = gemv_xr_kernel<FMT, CW>;
    static bool configured[64] = {};
    int dev = 0;
    B200Q_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        B200Q_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemMax));
        // the whole unified cache as shared memory, like the other GEMV kernels of a decode chain: a
        // different split would have to wait for the SM to drain before the next kernel could move in
        B200Q_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(CW * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = stream_get_option(1) ? 1 : 0;
    B200Q_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, p));
    *taken = true;
    return B200Q_OK;
}

int launch_gemv_xr(int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype, int M, int N, int K,
                   int sms, int* status, cudaStream_t st, bool* taken) {
    if (fmt == kQ6_K) return launch_gemv_xr_cw<kQ6_K, 16>(fmt, W, X, x_dtype, bias, Y, y_dtype, M, N, K, sms, status, st, taken);
    return launch_gemv_xr_cw<kQ4_K, 16>(fmt, W, X, x_dtype, bias, Y, y_dtype, M, N, K, sms, status, st, taken);
}

}  // namespace b200q

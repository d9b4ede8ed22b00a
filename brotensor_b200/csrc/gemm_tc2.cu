// Prefill GEMM on a CTA pair (thread-block cluster of two, tcgen05 cta_group::2):
//   Y(M,N) = X(M,K) * decode(W(N,K))^T (+bias), FP16 operands, FP32 accumulation in TMEM.
//
// Why a pair. With one CTA per 128 weight rows the activation operand of 512 tokens is
// re-streamed from L2 by every CTA at 64 KB per 64-k stage - at the MMA rate that is the
// whole L2->SM bandwidth of an SM, and only two such stages fit in shared memory, so the
// tensor pipe waits for operand data about half of the time. A pair of CTAs on two SMs runs
// ONE MMA of 256 weight rows (128 per CTA, each from its own shared memory and into its own
// TMEM) whose token operand is split between the two shared memories: each CTA fetches
// only half of the tokens (32 KB per stage), the slab ring becomes four stages deep, and
// every weight block is still decoded exactly once.
//
// Roles, identical in both CTAs unless noted:
//   warp 0   loader: bulk async copies of this CTA's half of the activation slabs;
//   warp 1   TMEM allocation; in the leader CTA (cluster rank 0) one thread of warp 1 and one
//            of warp 3 issue the MMAs of alternate stages and commit them to the stage
//            barriers of both CTAs;
//   warp 2   relay: tells the leader when this CTA's slab has landed (a bulk copy can only
//            signal a barrier of the CTA it writes to);
//   warps 4..11  decode this CTA's 128 weight rows into the A-operand ring (two threads per
//            row) and arrive on the LEADER's "A ready" barrier; afterwards the epilogue.
// All waits are bounded; on a timeout the CTA records a status code, stops working, still
// takes part in the cluster barriers, frees its TMEM and returns.
//
// Takes the place of brotensor's fused-dequant WMMA kernels (src/cuda/q4k_wmma.cu:56-310,
// q6k_wmma.cu:62-356, q8_0_wmma.cu:54-288).
#include "gemm_common.cuh"

namespace b200q {

constexpr int kPairCtrlWarps = 4;
constexpr int kPairProducerWarps = 8;
constexpr int kPairThreads = 32 * (kPairCtrlWarps + kPairProducerWarps);
constexpr int kPairMaxStages = 8;

struct PairParams {
    const uint8_t* W;
    const uint8_t* Xp;   // prepared activations of this pass: [K/64][tok_stride][64] FP16, swizzled rows
    const void* bias;
    void* Y;
    int* status;
    int tokens, tok_pad, xp_tok_stride;
    int N, K, row_bytes;
    int bias_dtype, y_dtype;
    int n_a, n_b;        // ring depths in k-blocks: decoded weights (16 KB slots) and slabs; n_b <= n_a
    int g_bytes;         // bytes of one token group's half in a slab slot: (min(tok_pad, 256) / 2) * 128
    int b_bytes;         // one slab slot of this CTA: g_bytes * groups
    // Split K (few row tiles, long rows): blockIdx.y = s works on k-blocks [s * kb_split, (s + 1) * kb_split) and
    // writes its FP32 partial sums, without bias, to Ypart[s][token][N]; a second kernel adds them up in order.
    int n_split, kb_split;
    size_t w_split_bytes;  // bytes of kb_split k-blocks of one weight row
    float* Ypart;
};

// ---- cluster / cta_group::2 wrappers ----------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of `saddr` (a shared::cta address of this CTA) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_to_rank(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrival on a barrier of another CTA of the cluster. Default (CTA-scope release) semantics on
// purpose: what has to be ordered before it is this CTA's own shared-memory image, which the
// proxy fence has already made visible to the tensor cores; a cluster-scope release here is a
// full memory barrier per producer warp and stage and cost a third of the kernel's time.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrives on the barrier at shared::cluster address `bar` once all MMAs issued so far have retired
__device__ __forceinline__ void umma2_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// kind::f16 instruction descriptor of the pair MMA: D = F32, A = B = F16, K-major, M = 256, N = n
__device__ __forceinline__ uint32_t instr_desc_pair(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

// Pair P of a Q4_K block: its 32 quant bytes hold sub-block 2P in the low nibbles (k 0..31 of the
// stage) and sub-block 2P+1 in the high ones (k 32..63). The row's two threads split the BYTES: thread
// half H holds bytes 16H .. 16H+15 of every pair (`blk[1 + P]`, beside the 16-byte header `blk[0]`),
// so together they load each byte of the block once, and H writes k 16H .. 16H+15 (16-byte chunks
// 2H, 2H+1 of the row) from the low nibbles and k 32+16H .. (chunks 4+2H, 5+2H) from the high ones.
template <int P>
__device__ __forceinline__ void q4k_split_to_smem(const uint4 (&blk)[5], uint32_t rowaddr, uint32_t r7, int H) {
    const uint4 h = blk[0];
    uint32_t sc0, m0, sc1, m1;
    if constexpr (P < 2) {
        sc0 = (h.y >> (16 * P)) & 63u;
        m0 = (h.z >> (16 * P)) & 63u;
        sc1 = (h.y >> (16 * P + 8)) & 63u;
        m1 = (h.z >> (16 * P + 8)) & 63u;
    } else {
        constexpr int J = 2 * (P - 2);
        sc0 = ((h.w >> (8 * J)) & 0xFu) | (((h.y >> (8 * J + 6)) & 3u) << 4);
        m0 = ((h.w >> (8 * J + 4)) & 0xFu) | (((h.z >> (8 * J + 6)) & 3u) << 4);
        sc1 = ((h.w >> (8 * J + 8)) & 0xFu) | (((h.y >> (8 * J + 14)) & 3u) << 4);
        m1 = ((h.w >> (8 * J + 12)) & 0xFu) | (((h.z >> (8 * J + 14)) & 3u) << 4);
    }
    const float d = h2f(h.x & 0xFFFFu), dmin = h2f(h.x >> 16);
    const float ds0 = d * (float)sc0, dm0 = dmin * (float)m0, ds1 = d * (float)sc1, dm1 = dmin * (float)m1;
    const uint4 q = blk[1 + P];
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        uint4 o;
        nib4_to_h2(w[2 * c] & 0x0F0F0F0Fu, ds0, dm0, o.x, o.y);
        nib4_to_h2(w[2 * c + 1] & 0x0F0F0F0Fu, ds0, dm0, o.z, o.w);
        sts128(rowaddr + (((uint32_t)(c + 2 * H) ^ r7) << 4), o);
    }
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        uint4 o;
        nib4_to_h2((w[2 * c] >> 4) & 0x0F0F0F0Fu, ds1, dm1, o.x, o.y);
        nib4_to_h2((w[2 * c + 1] >> 4) & 0x0F0F0F0Fu, ds1, dm1, o.z, o.w);
        sts128(rowaddr + (((uint32_t)(4 + c + 2 * H) ^ r7) << 4), o);
    }
}
// One Q8_0 block (FP16 d + 32 int8) held as the nine aligned words that cover it: an even block
// (H = 0) starts on word 0, its quants two bytes in; an odd block (H = 1) starts two bytes into
// word 0, so d is the high half of word 0 and the quants are words 1..8. The thread
// writes its 32 weights as 16-byte chunks 4H .. 4H+3 of the row: d * q is exact in FP32, one rounding.
__device__ __forceinline__ void q8_0_half_to_smem(const uint32_t (&w)[9], uint32_t rowaddr, uint32_t r7, int H) {
    const float d = h2f(H ? (w[0] >> 16) : (w[0] & 0xFFFFu));
    const uint32_t sh = 16u + 16u * (uint32_t)H;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const uint32_t q = __funnelshift_rc(w[2 * c + j], w[2 * c + j + 1], sh) ^ 0x80808080u;  // int8 + 128
            float f[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) f[i] = d * (__uint_as_float(__byte_perm(q, 0x4B000000u, 0x7440 | i)) - 8388736.0f);
            o[2 * j] = pack_h2(f[0], f[1]);
            o[2 * j + 1] = pack_h2(f[2], f[3]);
        }
        sts128(rowaddr + (((uint32_t)(c + 4 * H) ^ r7) << 4), make_uint4(o[0], o[1], o[2], o[3]));
    }
}
// One quad (32 elements) of a Q6_K block: `ql` its 32 nibble bytes (low nibbles for quads 0 and 1,
// high for 2 and 3), `qh` the group's 32 high-bit bytes (two bits per quad), `sc2` the quad's two
// int8 sub-block scales, `d16` the block's FP16 d. w = d * sc * (raw6 - 32): d * sc and the product
// with the 6-bit value are exact in FP32, one rounding to FP16. Written as chunks 4H .. 4H+3 of the row.
__device__ __forceinline__ void q6k_quad_to_smem(const uint32_t (&ql)[8], const uint32_t (&qh)[8], uint32_t sc2, uint32_t d16,
                                                 int quad, uint32_t rowaddr, uint32_t r7, int H) {
    const float d = h2f(d16 & 0xFFFFu);
    const float ds0 = d * (float)(int)(signed char)(sc2 & 0xFFu), ds1 = d * (float)(int)(signed char)((sc2 >> 8) & 0xFFu);
    const uint32_t nsh = quad >= 2 ? 4u : 0u, hsh = 2u * (uint32_t)quad;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const float ds = c < 2 ? ds0 : ds1;  // elements 0..15 / 16..31 of the quad
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const uint32_t v = ((ql[2 * c + j] >> nsh) & 0x0F0F0F0Fu) | (((qh[2 * c + j] >> hsh) & 0x03030303u) << 4);  // raw6, 0..63
            float f[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) f[i] = ds * (__uint_as_float(__byte_perm(v, 0x4B000000u, 0x7440 | i)) - 8388640.0f);  // 2^23 + 32
            o[2 * j] = pack_h2(f[0], f[1]);
            o[2 * j + 1] = pack_h2(f[2], f[3]);
        }
        sts128(rowaddr + (((uint32_t)(c + 4 * H) ^ r7) << 4), make_uint4(o[0], o[1], o[2], o[3]));
    }
}

template <int FMT>
__global__ void __launch_bounds__(kPairThreads, 1) gemm_tc2_kernel(const PairParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;  // operand tiles need 1024-byte alignment
    __shared__ uint64_t bar_ready[kPairMaxStages];    // leader: the k-block's operands are complete: both CTAs' producer
                                                      // warps have written their A slot and both slab halves have landed
    __shared__ uint64_t bar_a_empty[kPairMaxStages];  // the pair's MMAs on the k-block retired (commit from the leader)
    __shared__ uint64_t bar_b_full[kPairMaxStages];   // this CTA's half of the slab landed (tx)
    __shared__ uint64_t bar_turn[2];                  // leader: issuer q may queue its next stage (strict alternation)
    __shared__ uint64_t bar_accum;                    // all MMAs retired
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t crank = cluster_ctarank();         // 0 = leader
    const int row0 = blockIdx.x * kGemmRows;          // the pair's CTAs own consecutive row tiles
    const int n_kb = p.n_split > 1 ? p.kb_split : p.K / kBK;  // k-blocks of this CTA; its first one is blockIdx.y * kb_split
    const uint32_t tmem_cols = p.tok_pad <= 32 ? 32u : p.tok_pad <= 64 ? 64u : p.tok_pad <= 128 ? 128u : p.tok_pad <= 256 ? 256u : 512u;
    // token groups of up to 256: group g is one MMA of N = ng tokens into accumulator columns 256 g ..;
    // this CTA holds tokens [256 g + crank * ng / 2, + ng / 2) of it
    const int n0 = min(p.tok_pad, 256), n1 = p.tok_pad - n0;
    const int groups = n1 > 0 ? 2 : 1;

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < p.n_a; ++s) {
            mbar_init(smem_u32(&bar_ready[s]), 2 * kPairProducerWarps + 2);
            mbar_init(smem_u32(&bar_a_empty[s]), 1);
        }
        for (int s = 0; s < p.n_b; ++s) mbar_init(smem_u32(&bar_b_full[s]), 1);
        mbar_init(smem_u32(&bar_turn[0]), 1);
        mbar_init(smem_u32(&bar_turn[1]), 1);
        mbar_init(smem_u32(&bar_accum), 2);
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc2(smem_u32(&tmem_base_slot), tmem_cols);
        tmem_relinquish2();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    const uint32_t b_base = sbase + (uint32_t)(p.n_a * kGemmRows * 128);  // A ring first, then the slab ring

    if (warp == 0) {
        // ---- loader. The slab slot of k-block kb is free once the MMAs of k-block kb - n_b have
        // retired, which is what that k-block's A-slot barrier says (n_b <= n_a).
        if (lane == 0) {
            int bs = 0, sa = 0;
            uint32_t pa = 0;
            for (int kb = 0; kb < n_kb; ++kb) {
                if (kb >= p.n_b) {
                    if (!wait_or_abort<true>(smem_u32(&bar_a_empty[sa]), pa, &abort_flag, p.status, kDevTimeoutEmpty)) break;
                    if (++sa == p.n_a) { sa = 0; pa ^= 1; }
                }
                const uint32_t full = smem_u32(&bar_b_full[bs]);
                const uint32_t h0 = (uint32_t)(n0 / 2) * 128u, h1 = (uint32_t)(n1 / 2) * 128u;
                mbar_arrive_expect_tx(full, h0 + h1);
                const uint8_t* src = p.Xp + (size_t)(kb + (int)blockIdx.y * p.kb_split) * p.xp_tok_stride * 128u;
                const uint32_t dst = b_base + bs * p.b_bytes;
                bulk_g2s(dst, src + (size_t)crank * h0, h0, full);
                if (groups == 2) bulk_g2s(dst + p.g_bytes, src + 256u * 128u + (size_t)crank * h1, h1, full);
                if (++bs == p.n_b) bs = 0;
            }
        }
    } else if (warp == 2) {
        // ---- relay: this CTA's half has landed -> one arrival on the leader's "ready" barrier of the k-block
        if (lane == 0) {
            int bs = 0, sa = 0;
            uint32_t pb = 0;
            for (int kb = 0; kb < n_kb; ++kb) {
                if (!wait_or_abort<true>(smem_u32(&bar_b_full[bs]), pb, &abort_flag, p.status, kDevTimeoutFull)) break;
                mbar_arrive_remote(map_to_rank(smem_u32(&bar_ready[sa]), 0));
                if (++bs == p.n_b) { bs = 0; pb ^= 1; }
                if (++sa == p.n_a) sa = 0;
            }
        }
    } else if (warp == 1 || warp == 3) {
        // ---- MMA issuers (leader CTA only). One thread cannot keep the tensor pipe fed: issuing
        // blocks while the pipe's short queue is full, and the wait / fence / commits between two
        // stages would then leave it idle. Two threads in different warps take alternate stages:
        // while one is blocked behind its own MMAs, the other has done the next stage's wait and
        // queues up right behind it. A turn barrier keeps the queueing order kb = 0, 1, 2, ...
        // so the accumulation order, and with it the result, is the same on every run.
        if (lane == 0 && crank == 0) {
            const int q = warp == 1 ? 0 : 1;
            int sa = q % p.n_a, bs = q % p.n_b;
            uint32_t pa = (uint32_t)(q / p.n_a) & 1u, pt = 0;
            const uint32_t idesc0 = instr_desc_pair(n0), idesc1 = instr_desc_pair(n1 > 0 ? n1 : 16);
            for (int kb = q; kb < n_kb; kb += 2) {
                if (!wait_or_abort<true>(smem_u32(&bar_ready[sa]), pa, &abort_flag, p.status, kDevTimeoutFull)) break;
                if (kb > 0) {  // my turn: the other issuer has queued stage kb - 1
                    if (!wait_or_abort<true>(smem_u32(&bar_turn[q]), pt, &abort_flag, p.status, kDevTimeoutFull)) break;
                    pt ^= 1;
                }
                tc_fence_after();
                const uint32_t a_s = sbase + sa * (kGemmRows * 128), b_s = b_base + bs * p.b_bytes;
#pragma unroll
                for (int k = 0; k < kBK / 16; ++k) {
                    const uint64_t adesc = smem_desc_sw128(a_s + k * 32);
                    umma2_f16(tmem_base, adesc, smem_desc_sw128(b_s + k * 32), idesc0, (kb | k) != 0);
                    if (groups == 2) umma2_f16(tmem_base + 256, adesc, smem_desc_sw128(b_s + p.g_bytes + k * 32), idesc1, (kb | k) != 0);
                }
                mbar_arrive(smem_u32(&bar_turn[q ^ 1]));
                // the k-block's A slots (and, n_b k-blocks on, its slabs) are free in both CTAs once these have retired
                umma2_commit(smem_u32(&bar_a_empty[sa]));
                umma2_commit(map_to_rank(smem_u32(&bar_a_empty[sa]), 1));
                sa += 2;
                if (sa >= p.n_a) { sa -= p.n_a; pa ^= 1; }
                bs += 2;
                if (bs >= p.n_b) bs -= p.n_b;
            }
            umma2_commit(smem_u32(&bar_accum));
            umma2_commit(map_to_rank(smem_u32(&bar_accum), 1));
        }
    } else if (warp >= kPairCtrlWarps) {
        // ---- A producers (two threads per weight row: k 0..31 and k 32..63 of the stage), then the epilogue
        const int H = (warp - kPairCtrlWarps) >> 2;
        const int pt = (warp & 3) * 32 + lane;                   // tile row = TMEM lane of this thread
        const int wrow = min(row0 + pt, p.N - 1);                // rows past N decode row N-1, never stored
        const uint8_t* rowp = p.W + (size_t)wrow * p.row_bytes + (size_t)blockIdx.y * p.w_split_bytes;
        const uint32_t r7 = (uint32_t)(pt & 7);
        const uint32_t row_off = (uint32_t)((pt >> 3) * 1024 + (pt & 7) * 128);
        const int n_blk = n_kb / 4;  // blocks of this CTA's k range (the prefetch must not run past it: the last row ends there)
        int slot = 0, prev_slot = 0;
        uint32_t phase = 0;
        bool live = true;
        // This thread's share of the row's Q4_K block for the next four stages (the header and bytes
        // 16H .. 16H+15 of each of the four 32-byte pairs) is loaded into registers one block ahead
        // of its use, so its latency (an L2 or DRAM round trip) hides behind four stages of decode.
        uint4 cur[5], nxt[5];
#pragma unroll
        for (int i = 0; i < 5; ++i) cur[i] = nxt[i] = make_uint4(0, 0, 0, 0);
        auto q4_load = [&](int b, uint4 (&dst)[5]) {
            const uint4* src = reinterpret_cast<const uint4*>(rowp + (size_t)b * 144);
            dst[0] = __ldg(src);
#pragma unroll
            for (int i = 0; i < 4; ++i) dst[1 + i] = __ldg(src + 1 + 2 * i + H);
        };
        if constexpr (FMT == kQ4_K) q4_load(0, nxt);
        // Q8_0: eight blocks (256 k, 272 bytes = 17 x 16) form a 16-byte aligned chunk. The thread's
        // block of stage P = kb & 3 is block 2P + H of the chunk: it lies inside the three 16-byte
        // words 4P + 2H .. +2, starting at byte 4P + 2H of them. They are loaded one stage ahead.
        uint4 c8[3], c8n[3];
        auto q8_load = [&](int kbb, uint4 (&dst)[3]) {
            const uint4* src = reinterpret_cast<const uint4*>(rowp + (size_t)(kbb >> 2) * 272) + 4 * (kbb & 3) + 2 * H;
#pragma unroll
            for (int i = 0; i < 3; ++i) dst[i] = __ldg(src + i);
        };
#pragma unroll
        for (int i = 0; i < 3; ++i) c8[i] = c8n[i] = make_uint4(0, 0, 0, 0);
        if constexpr (FMT == kQ8_0) q8_load(0, c8n);
        // Q6_K: the thread's two quads of the next PAIR of stages, loaded one pair ahead. Stages 2j and
        // 2j + 1 of a block decode quads H and 2 + H of group j: the low and the high nibbles of the
        // same 32 bytes, and two bit pairs of the same 32 high-bit bytes - loaded once for both (loaded
        // per stage, these reads, 3.7 times the bytes a stage holds, were most of the L2 -> SM traffic
        // beside the activation slabs, and that traffic is what bounds the kernel). Blocks are 210
        // bytes and only 2-byte aligned: the 32 nibble bytes and the 32 high-bit bytes are read
        // as three 16-byte words each from the 16-byte boundary at or before the block (both
        // regions start on a multiple of 32 bytes inside the block, so 48 bytes from the boundary
        // cover them for any alignment); `f6` keeps the block's byte offset from that boundary.
        // `S` holds the scales of quad H in its low half and those of quad 2 + H in its high half.
        uint4 l6[3], h6[3], l6n[3], h6n[3];
        uint32_t s6 = 0, d6 = 0, f6 = 0, s6n = 0, d6n = 0, f6n = 0;
        auto q6_load = [&](int kbb, uint4 (&L)[3], uint4 (&Hh)[3], uint32_t& S, uint32_t& D, uint32_t& F) {
            const int blk = kbb >> 2, grp = (kbb & 3) >> 1;  // kbb is even
            if constexpr (FMT == kQ6_KP) {
                // regrouped by field in runs of eight blocks: both 32-byte pieces are 16-byte aligned
                const uint8_t* run = rowp + (size_t)(blk >> 3) * kQ6RunBytes;
                const int s = blk & 7;
                const uint4* al = reinterpret_cast<const uint4*>(run + s * 128 + 64 * grp + 32 * H);
                const uint4* ah = reinterpret_cast<const uint4*>(run + 1024 + s * 64 + 32 * grp);
                L[0] = __ldg(al); L[1] = __ldg(al + 1);
                Hh[0] = __ldg(ah); Hh[1] = __ldg(ah + 1);
                S = (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(run + 1536 + s * 16 + grp * 8 + H * 2)) |
                    (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(run + 1536 + s * 16 + grp * 8 + 4 + H * 2)) << 16;
                D = __ldg(reinterpret_cast<const unsigned short*>(run + 1664 + 2 * s));
                F = 0;
                return;
            }
            const uint8_t* b0 = rowp + (size_t)blk * 210;
            F = (uint32_t)(reinterpret_cast<uintptr_t>(b0) & 15u);
            const uint4* al = reinterpret_cast<const uint4*>(b0 - F);
#pragma unroll
            for (int i = 0; i < 3; ++i) L[i] = __ldg(al + 4 * grp + 2 * H + i);
#pragma unroll
            for (int i = 0; i < 3; ++i) Hh[i] = __ldg(al + 8 + 2 * grp + i);
            S = (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(b0 + 192 + grp * 8 + H * 2)) |
                (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(b0 + 192 + grp * 8 + 4 + H * 2)) << 16;
            D = __ldg(reinterpret_cast<const unsigned short*>(b0 + 208));
        };
#pragma unroll
        for (int i = 0; i < 3; ++i) l6[i] = h6[i] = l6n[i] = h6n[i] = make_uint4(0, 0, 0, 0);
        const int kb0 = (int)blockIdx.y * p.kb_split;  // Q6_K addresses its blocks by the k-block's number in the whole row
        if constexpr (FMT == kQ6_K || FMT == kQ6_KP) q6_load(kb0, l6n, h6n, s6n, d6n, f6n);
        for (int kb = 0; kb < n_kb; ++kb) {
            if constexpr (FMT == kQ6_K || FMT == kQ6_KP) {
                if ((kb & 1) == 0) {
#pragma unroll
                    for (int i = 0; i < 3; ++i) { l6[i] = l6n[i]; h6[i] = h6n[i]; }
                    s6 = s6n; d6 = d6n; f6 = f6n;
                    if (kb + 2 < n_kb) q6_load(kb0 + kb + 2, l6n, h6n, s6n, d6n, f6n);
                }
            }
            if constexpr (FMT == kQ8_0) {
#pragma unroll
                for (int i = 0; i < 3; ++i) c8[i] = c8n[i];
                if (kb + 1 < n_kb) q8_load(kb + 1, c8n);
            }
            if constexpr (FMT == kQ4_K) {
                if ((kb & 3) == 0) {
                    const int b = kb >> 2;
#pragma unroll
                    for (int i = 0; i < 5; ++i) cur[i] = nxt[i];
                    if (b + 1 < n_blk) q4_load(b + 1, nxt);
                }
            }
            if (live) {
                const bool ok = gemm_wait(smem_u32(&bar_a_empty[slot]), phase ^ 1, &abort_flag, p.status, kDevTimeoutEmpty);
                live = __all_sync(0xffffffffu, ok);
            }
            if (live) {
                const uint32_t rowaddr = sbase + slot * (kGemmRows * 128) + row_off;
                if constexpr (FMT == kQ4_K) {
                    switch (kb & 3) {
                        case 0: q4k_split_to_smem<0>(cur, rowaddr, r7, H); break;
                        case 1: q4k_split_to_smem<1>(cur, rowaddr, r7, H); break;
                        case 2: q4k_split_to_smem<2>(cur, rowaddr, r7, H); break;
                        default: q4k_split_to_smem<3>(cur, rowaddr, r7, H); break;
                    }
                } else if constexpr (FMT == kQ8_0) {
                    const uint32_t w12[12] = {c8[0].x, c8[0].y, c8[0].z, c8[0].w, c8[1].x, c8[1].y, c8[1].z, c8[1].w,
                                              c8[2].x, c8[2].y, c8[2].z, c8[2].w};
                    // the block starts in word P of the twelve: on it for H = 0, two bytes into it for H = 1
                    uint32_t w9[9];
                    switch (kb & 3) {
                        case 0: for (int i = 0; i < 9; ++i) w9[i] = w12[i]; break;
                        case 1: for (int i = 0; i < 9; ++i) w9[i] = w12[1 + i]; break;
                        case 2: for (int i = 0; i < 9; ++i) w9[i] = w12[2 + i]; break;
                        default: for (int i = 0; i < 9; ++i) w9[i] = w12[3 + i]; break;
                    }
                    q8_0_half_to_smem(w9, rowaddr, r7, H);
                } else {
                    const uint32_t wl[12] = {l6[0].x, l6[0].y, l6[0].z, l6[0].w, l6[1].x, l6[1].y, l6[1].z, l6[1].w,
                                             l6[2].x, l6[2].y, l6[2].z, l6[2].w};
                    const uint32_t wh[12] = {h6[0].x, h6[0].y, h6[0].z, h6[0].w, h6[1].x, h6[1].y, h6[1].z, h6[1].w,
                                             h6[2].x, h6[2].y, h6[2].z, h6[2].w};
                    // the data starts f6 bytes (even, 0..14) into the twelve words: whole words by the
                    // switch (the same for every lane when rows are a multiple of 16 bytes), two bytes by the shift
                    const uint32_t bits = (f6 & 2u) * 8u;
                    uint32_t ql[8], qh[8];
                    if constexpr (FMT == kQ6_KP) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) { ql[i] = wl[i]; qh[i] = wh[i]; }
                    } else
                    switch (f6 >> 2) {
                        case 0: for (int i = 0; i < 8; ++i) { ql[i] = __funnelshift_r(wl[i], wl[i + 1], bits); qh[i] = __funnelshift_r(wh[i], wh[i + 1], bits); } break;
                        case 1: for (int i = 0; i < 8; ++i) { ql[i] = __funnelshift_r(wl[1 + i], wl[2 + i], bits); qh[i] = __funnelshift_r(wh[1 + i], wh[2 + i], bits); } break;
                        case 2: for (int i = 0; i < 8; ++i) { ql[i] = __funnelshift_r(wl[2 + i], wl[3 + i], bits); qh[i] = __funnelshift_r(wh[2 + i], wh[3 + i], bits); } break;
                        default: for (int i = 0; i < 8; ++i) { ql[i] = __funnelshift_r(wl[3 + i], wl[4 + i], bits); qh[i] = __funnelshift_r(wh[3 + i], wh[4 + i], bits); } break;
                    }
                    q6k_quad_to_smem(ql, qh, (kb & 1) ? s6 >> 16 : s6, d6, 2 * (kb & 1) + H, rowaddr, r7, H);
                }
            }
            // One proxy fence and one warp synchronisation for two k-blocks (their number is even): measured 2 % on
            // the 512-token shapes of Q4_K and Q6_K (60.8 against 62.4 us, 79.5 against 81.0 on one box), nothing
            // where the decode alone sets the pace (32 tokens).
            if (kb & 1) {
                if (live) fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor cores of the pair
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive_remote(map_to_rank(smem_u32(&bar_ready[prev_slot]), 0));
                    mbar_arrive_remote(map_to_rank(smem_u32(&bar_ready[slot]), 0));
                }
            } else {
                prev_slot = slot;
            }
            if (++slot == p.n_a) { slot = 0; phase ^= 1; }
        }
        // ---- epilogue: this CTA's accumulator rows are its own 128 weight rows; a warp may only
        // touch TMEM lanes 32*(warp%4)..+31, and the two warps sharing a lane quarter split the tokens
        if (live) {
            const bool ok = gemm_wait(smem_u32(&bar_accum), 0, &abort_flag, p.status, kDevTimeoutMma);
            live = __all_sync(0xffffffffu, ok);
        }
        if (live) {
            tc_fence_after();
            const int n = row0 + pt;
            float bv = 0.f;
            if (p.bias && n < p.N) {
                if (p.bias_dtype == B200Q_DT_F32) bv = static_cast<const float*>(p.bias)[n];
                else if (p.bias_dtype == B200Q_DT_F16) bv = __half2float(static_cast<const __half*>(p.bias)[n]);
                else bv = __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[n]);
            }
            const uint32_t tlane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
            const int share = ((p.tok_pad / 16 + 1) / 2) * 16;
            const int cbeg = H * share, cend = min(cbeg + share, p.tok_pad);
            for (int c0 = cbeg; c0 < cend; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(tlane + (uint32_t)c0, r);
                tmem_ld_wait();
                if (n < p.N && p.n_split > 1) {
                    float* part = p.Ypart + (size_t)blockIdx.y * p.tokens * p.N;
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (c0 + j < p.tokens) part[(size_t)(c0 + j) * p.N + n] = __uint_as_float(r[j]);
                } else if (n < p.N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int t = c0 + j;
                        if (t < p.tokens) {
                            const float v = __uint_as_float(r[j]) + bv;
                            const size_t o = (size_t)t * p.N + n;
                            if (p.y_dtype == B200Q_DT_F32) static_cast<float*>(p.Y)[o] = v;
                            else if (p.y_dtype == B200Q_DT_F16) static_cast<__half*>(p.Y)[o] = __float2half_rn(v);
                            else static_cast<__nv_bfloat16*>(p.Y)[o] = __float2bfloat16_rn(v);
                        }
                    }
                }
            }
        }
    }
    // Nobody leaves (or frees TMEM) while the other CTA may still read this one's shared memory,
    // arrive on its barriers or have MMAs of the pair in flight.
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc2(tmem_base, tmem_cols);
    }
}

// ---- host side ---------------------------------------------------------------------------------

template <int FMT>
static int launch_pair_fmt(const PairParams& p, size_t smem, cudaStream_t st) {
    auto kern = gemm_tc2_kernel<FMT>;
    static bool configured[64] = {};
    int dev = 0;
    B200Q_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        B200Q_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 1024));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const unsigned tiles = (unsigned)((p.N + kGemmRows - 1) / kGemmRows);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((tiles + 1u) & ~1u, (unsigned)(p.n_split > 1 ? p.n_split : 1));  // whole pairs; a CTA past the last row tile decodes row N-1 and stores nothing
    cfg.blockDim = dim3(kPairThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B200Q_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, p));
    return B200Q_OK;
}

// Y[t][n] = bias[n] + part[0][t][n] + part[1][t][n] + ... in that order (the same on every run), four
// neighbouring n per thread.
__global__ void __launch_bounds__(256) gemm_split_reduce_kernel(const float* __restrict__ part, int n_split, int tokens, int N,
                                                                const void* __restrict__ bias, int bias_dtype, void* __restrict__ Y, int y_dtype) {
    const size_t total = (size_t)tokens * N, quads = total / 4;  // N % 4 == 0 is checked by the caller
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += (size_t)gridDim.x * blockDim.x) {
        const int n = (int)((4 * i) % (size_t)N);
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        if (bias) {
            if (bias_dtype == B200Q_DT_F32) a = *reinterpret_cast<const float4*>(static_cast<const float*>(bias) + n);
            else if (bias_dtype == B200Q_DT_F16) {
                const __half* b = static_cast<const __half*>(bias) + n;
                a = make_float4(__half2float(b[0]), __half2float(b[1]), __half2float(b[2]), __half2float(b[3]));
            } else {
                const __nv_bfloat16* b = static_cast<const __nv_bfloat16*>(bias) + n;
                a = make_float4(__bfloat162float(b[0]), __bfloat162float(b[1]), __bfloat162float(b[2]), __bfloat162float(b[3]));
            }
        }
        // the tensor cores' sum of a split first, then the bias: with one split this is the order of the unsplit epilogue
        float4 sum = __ldcs(reinterpret_cast<const float4*>(part) + i);
        for (int s = 1; s < n_split; ++s) {
            const float4 v = __ldcs(reinterpret_cast<const float4*>(part + (size_t)s * total) + i);
            sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
        }
        sum.x += a.x; sum.y += a.y; sum.z += a.z; sum.w += a.w;
        if (y_dtype == B200Q_DT_F32) reinterpret_cast<float4*>(Y)[i] = sum;
        else if (y_dtype == B200Q_DT_F16) {
            __half2* y = reinterpret_cast<__half2*>(Y) + 2 * i;
            y[0] = __floats2half2_rn(sum.x, sum.y);
            y[1] = __floats2half2_rn(sum.z, sum.w);
        } else {
            __nv_bfloat162* y = reinterpret_cast<__nv_bfloat162*>(Y) + 2 * i;
            y[0] = __floats2bfloat162_rn(sum.x, sum.y);
            y[1] = __floats2bfloat162_rn(sum.z, sum.w);
        }
    }
}

// One pass (<= 512 tokens) of the prefill GEMM on CTA pairs. The caller has run the activation
// pre-pass; Xp points at this pass's first token row inside the workspace. n_split > 1: K is split
// over blockIdx.y and `ypart` (n_split * tokens * N floats) takes the partial sums.
int launch_gemm_pair_pass(int fmt, const void* W, const uint8_t* Xp, int tok_stride, const void* bias, int bias_dtype,
                          void* Y, int y_dtype, int tokens, int N, int K, int n_split, float* ypart, int* status, cudaStream_t st) {
    PairParams p = {};
    p.n_split = n_split > 1 ? n_split : 1;
    p.kb_split = (K / kBK) / p.n_split;
    // (the Q6_K producers find a block from the k-block's number in the whole row - the regrouped layout has no
    // per-split row offset - so their row pointer stays put)
    p.w_split_bytes = (fmt == kQ6_K || fmt == kQ6_KP) ? 0 : (size_t)(p.kb_split * kBK / b200q_block_elems(fmt)) * b200q_block_bytes(fmt);
    p.Ypart = ypart;
    p.W = static_cast<const uint8_t*>(W);
    p.Xp = Xp;
    p.bias = bias;
    p.Y = Y;
    p.status = status;
    p.tokens = tokens;
    p.tok_pad = (tokens + 15) & ~15;
    p.xp_tok_stride = tok_stride;
    p.N = N;
    p.K = K;
    p.row_bytes = (K / b200q_block_elems(fmt)) * b200q_block_bytes(fmt);
    p.bias_dtype = bias_dtype;
    p.y_dtype = y_dtype;
    const int n0 = p.tok_pad < 256 ? p.tok_pad : 256;
    const int groups = p.tok_pad > 256 ? 2 : 1;
    p.g_bytes = (n0 / 2) * 128;
    p.b_bytes = p.g_bytes * groups;
    // Ring depths: slabs three k-blocks ahead (they come from L2 with about a microsecond of latency), decoded
    // weights in the rest - of 196 KB, not of all the shared memory an SM has: what the kernel leaves of the
    // 256 KB array is the L1 its producers' weight loads go through, and the carve-out steps from 196 KB to the
    // full size at once. With 224 KB of rings (6 + 4 slots at 512 tokens) the L1 is ~28 KB and the Q6_K
    // producers, whose rows advance through 27 KB per block step, miss in it: Q6_K 85.4 us, its regrouped
    // layout 89.0; with 192 KB (6 + 3) 81.7 and 68.5; Q4_K 59.7 -> 59.1, Q8_0 67.5 -> 66.2 (512 x 14336 x 4096,
    // one box). Two slabs cost Q4_K 12 us, fewer than five weight slots 2.
    const unsigned budget = 196u * 1024u - 2048u;
    const unsigned kb_a = kGemmRows * 128;
    p.n_b = 3;
    p.n_a = (int)((budget - (unsigned)p.n_b * (unsigned)p.b_bytes) / kb_a);
    if (p.n_a > kPairMaxStages) p.n_a = kPairMaxStages;
    if (p.n_a < p.n_b) return fail(B200Q_ERR_UNSUPPORTED, "gemm: pair rings do not fit (%d weight slots, %d slab stages)", p.n_a, p.n_b);
    const size_t smem = (size_t)p.n_a * kb_a + (size_t)p.n_b * p.b_bytes + 1024;
    int rc;
    if (fmt == kQ4_K) rc = launch_pair_fmt<kQ4_K>(p, smem, st);
    else if (fmt == kQ6_K) rc = launch_pair_fmt<kQ6_K>(p, smem, st);
    else if (fmt == kQ6_KP) rc = launch_pair_fmt<kQ6_KP>(p, smem, st);
    else rc = launch_pair_fmt<kQ8_0>(p, smem, st);
    if (rc || p.n_split == 1) return rc;
    const size_t quads = (size_t)tokens * N / 4;
    size_t blocks = (quads + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    gemm_split_reduce_kernel<<<(unsigned)blocks, 256, 0, st>>>(ypart, p.n_split, tokens, N, bias, bias_dtype, Y, y_dtype);
    B200Q_CUDA_TRY(cudaGetLastError());
    return B200Q_OK;
}

}  // namespace b200q

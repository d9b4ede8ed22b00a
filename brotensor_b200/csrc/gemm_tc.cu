// Prefill GEMM on the 5th-generation tensor cores (sm_100a):
//   Y(M,N) = X(M,K) * decode(W(N,K))^T (+bias), FP16 operands, FP32 accumulation in TMEM.
//
// One CTA owns 128 weight rows and up to 512 activation rows (tokens), so every weight
// block is decoded exactly once per pass:
//   * the activations are converted once, by a small pre-pass, to FP16 in the exact
//     shared-memory image the MMA wants (K-major rows of 64 values = 128 bytes, 128-byte
//     swizzle) and kept in a caller-provided workspace, so a stage's whole B operand
//     (tokens x 64 k) is one contiguous range fetched with 1-D bulk async copies;
//   * four producer warps (one thread per weight row) decode 64 weights per stage to
//     FP16 - the FP32 decode is exact and is rounded once, like the reference's
//     __float2half_rn - and write the A operand in the same swizzled layout;
//   * one thread issues tcgen05.mma (M=128, N<=256 per instruction, K=16) into one or
//     two TMEM accumulators of 256 columns; tcgen05.commit releases the stage;
//   * the producer warps then read the accumulators back with tcgen05.ld, add the bias
//     and store Y, 32 consecutive outputs of a token per warp store.
// All waits are bounded; on a timeout the kernel records a status code, skips the rest of
// its work, still frees its TMEM and returns.
//
// Takes the place of brotensor's fused-dequant WMMA kernels (src/cuda/q4k_wmma.cu:56-310,
// q6k_wmma.cu:62-356, q8_0_wmma.cu:54-288: 64x64x32 tiles, wmma m16n16k16, single-buffered).
#include "stream_common.cuh"

namespace b200q {

constexpr int kGemmThreads = 192;        // warp 0: B loader, warp 1: MMA issuer + TMEM, warps 2..5: A producers / epilogue
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

template <int FMT>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_tc_kernel(const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;  // operand tiles need 1024-byte alignment
    __shared__ uint64_t bar_full[kGemmMaxStages];   // A written (4 producer warps) + B landed (tx)
    __shared__ uint64_t bar_empty[kGemmMaxStages];  // MMAs of the stage retired (tcgen05.commit)
    __shared__ uint64_t bar_accum;                  // all MMAs retired
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row0 = blockIdx.x * kGemmRows;
    const int n_kb = p.K / kBK;
    const uint32_t tmem_cols = p.tok_pad <= 32 ? 32u : p.tok_pad <= 64 ? 64u : p.tok_pad <= 128 ? 128u : p.tok_pad <= 256 ? 256u : 512u;

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < p.n_stages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 5);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        mbar_init(smem_u32(&bar_accum), 1);
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        // ---- B loader: the stage's activations are one contiguous range of the workspace
        if (lane == 0) {
            int slot = 0;
            uint32_t phase = 0;
            const uint32_t bbytes = (uint32_t)p.tok_pad * 128u;
            for (int kb = 0; kb < n_kb; ++kb) {
                if (!gemm_wait(smem_u32(&bar_empty[slot]), phase ^ 1, &abort_flag, p.status, kDevTimeoutEmpty)) break;
                const uint32_t full = smem_u32(&bar_full[slot]);
                mbar_arrive_expect_tx(full, bbytes);
                const uint8_t* src = p.Xp + (size_t)kb * p.xp_tok_stride * 128u;
                const uint32_t dst = sbase + slot * p.stage_bytes + kGemmRows * 128;
                for (uint32_t off = 0; off < bbytes; off += 32768u)
                    bulk_g2s(dst + off, src + off, min(32768u, bbytes - off), full);
                if (++slot == p.n_stages) { slot = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer
        if (lane == 0) {
            int slot = 0;
            uint32_t phase = 0;
            const int n0 = min(p.tok_pad, 256), n1 = p.tok_pad - n0;
            const uint32_t idesc0 = instr_desc_f16(n0), idesc1 = instr_desc_f16(n1 > 0 ? n1 : 16);
            bool ok = true;
            for (int kb = 0; kb < n_kb && ok; ++kb) {
                ok = gemm_wait(smem_u32(&bar_full[slot]), phase, &abort_flag, p.status, kDevTimeoutFull);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_s = sbase + slot * p.stage_bytes, b_s = a_s + kGemmRows * 128;
#pragma unroll
                for (int k = 0; k < kBK / 16; ++k) {
                    const uint64_t adesc = smem_desc_sw128(a_s + k * 32);
                    umma_f16(tmem_base, adesc, smem_desc_sw128(b_s + k * 32), idesc0, (kb | k) != 0);
                    if (n1 > 0) umma_f16(tmem_base + 256, adesc, smem_desc_sw128(b_s + 256 * 128 + k * 32), idesc1, (kb | k) != 0);
                }
                umma_commit(smem_u32(&bar_empty[slot]));  // frees the stage when these MMAs have read it
                if (++slot == p.n_stages) { slot = 0; phase ^= 1; }
            }
            umma_commit(smem_u32(&bar_accum));
        }
    } else {
        // ---- A producers (one thread per weight row), then the epilogue
        const int pt = (warp - 2) * 32 + lane;                   // 0..127: tile row this thread decodes
        const int wrow = min(row0 + pt, p.N - 1);                // rows past N decode row N-1, never stored
        const uint8_t* rowp = p.W + (size_t)wrow * p.row_bytes;
        const uint32_t r7 = (uint32_t)(pt & 7);
        const uint32_t row_off = (uint32_t)((pt >> 3) * 1024 + (pt & 7) * 128);
        int slot = 0;
        uint32_t phase = 0;
        bool live = true;
        uint4 cur[9], nxt[9];
        if constexpr (FMT == kQ4_K) {
#pragma unroll
            for (int i = 0; i < 9; ++i) cur[i] = __ldg(reinterpret_cast<const uint4*>(rowp) + i);
        }
        for (int kb = 0; kb < n_kb; ++kb) {
            if constexpr (FMT == kQ4_K) {
                if ((kb & 3) == 0 && kb + 4 < n_kb) {  // next block's 144 bytes, one block ahead of its use
#pragma unroll
                    for (int i = 0; i < 9; ++i) nxt[i] = __ldg(reinterpret_cast<const uint4*>(rowp + (size_t)((kb >> 2) + 1) * 144) + i);
                }
            }
            if (live) {
                const bool ok = gemm_wait(smem_u32(&bar_empty[slot]), phase ^ 1, &abort_flag, p.status, kDevTimeoutEmpty);
                live = __all_sync(0xffffffffu, ok);
            }
            if (live) {
                const uint32_t rowaddr = sbase + slot * p.stage_bytes + row_off;
                if constexpr (FMT == kQ4_K) {
                    switch (kb & 3) {
                        case 0: q4k_pair_to_smem<0>(cur, rowaddr, r7); break;
                        case 1: q4k_pair_to_smem<1>(cur, rowaddr, r7); break;
                        case 2: q4k_pair_to_smem<2>(cur, rowaddr, r7); break;
                        default: q4k_pair_to_smem<3>(cur, rowaddr, r7); break;
                    }
                } else {
                    generic_kb_to_smem<FMT>(rowp, kb, rowaddr, r7);
                }
                fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core's async proxy
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_full[slot]));
            if constexpr (FMT == kQ4_K) {
                if ((kb & 3) == 3) {
#pragma unroll
                    for (int i = 0; i < 9; ++i) cur[i] = nxt[i];
                }
            }
            if (++slot == p.n_stages) { slot = 0; phase ^= 1; }
        }
        // ---- epilogue: TMEM lane = weight row; a warp may only touch lanes 32*(warp%4)..+31
        if (live) {
            const bool ok = gemm_wait(smem_u32(&bar_accum), 0, &abort_flag, p.status, kDevTimeoutMma);
            live = __all_sync(0xffffffffu, ok);
        }
        if (live) {
            tc_fence_after();
            const int lrow = (warp & 3) * 32 + lane;
            const int n = row0 + lrow;
            float bv = 0.f;
            if (p.bias && n < p.N) {
                if (p.bias_dtype == B200Q_DT_F32) bv = static_cast<const float*>(p.bias)[n];
                else if (p.bias_dtype == B200Q_DT_F16) bv = __half2float(static_cast<const __half*>(p.bias)[n]);
                else bv = __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[n]);
            }
            const uint32_t tlane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
            for (int c0 = 0; c0 < p.tok_pad; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(tlane + (uint32_t)c0, r);
                tmem_ld_wait();
                if (n < p.N) {
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
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc(tmem_base, tmem_cols);
    }
}

// ---- host side ---------------------------------------------------------------------------------

static int round_up16(int v) { return (v + 15) & ~15; }

static bool gemm_tc_takes(int fmt, const void* W, int M, int K) {
    if (M <= 8) return false;                 // small batches stream the weight through the decode GEMV
    if (K % 256 != 0) return false;
    if (fmt == kQ4_K && (reinterpret_cast<uintptr_t>(W) & 15) != 0) return false;  // 16-byte block loads
    return fmt == kQ4_K || fmt == kQ6_K || fmt == kQ8_0;
}

size_t gemm_tc_workspace_bytes(int fmt, int x_dtype, int M, int N, int K) {
    (void)x_dtype; (void)N;
    if (!gemm_tc_takes(fmt, nullptr, M, K)) return 0;
    return (size_t)(K / kBK) * (size_t)round_up16(M) * 128u;
}

template <int FMT>
static int launch_gemm_fmt(const GemmParams& p, size_t smem, cudaStream_t st) {
    auto kern = gemm_tc_kernel<FMT>;
    static bool configured[64] = {};
    int dev = 0;
    B200Q_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        B200Q_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 1024));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const unsigned grid = (unsigned)((p.N + kGemmRows - 1) / kGemmRows);
    kern<<<grid, kGemmThreads, smem, st>>>(p);
    B200Q_CUDA_TRY(cudaGetLastError());
    return B200Q_OK;
}

int launch_gemm_tc(int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype, int M,
                   int N, int K, void* ws, size_t ws_bytes, int sms, int* status, cudaStream_t st, bool* taken) {
    (void)sms;
    *taken = gemm_tc_takes(fmt, W, M, K);
    if (!*taken) return B200Q_OK;
    const size_t need = gemm_tc_workspace_bytes(fmt, x_dtype, M, N, K);
    if (!ws || ws_bytes < need) return fail(B200Q_ERR_WORKSPACE, "gemm: workspace of %zu bytes needed, %zu given", need, ws ? ws_bytes : (size_t)0);
    if (reinterpret_cast<uintptr_t>(ws) & 255) return fail(B200Q_ERR_WORKSPACE, "gemm: workspace must be 256-byte aligned");
    const int tok_total = round_up16(M);
    {
        const long long total = (long long)(K / kBK) * tok_total * 8;
        long long blocks = (total + 255) / 256;
        if (blocks > 148LL * 16) blocks = 148LL * 16;
        uint4* xp = static_cast<uint4*>(ws);
        if (x_dtype == B200Q_DT_F32) gemm_xprep_kernel<float><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const float*>(X), xp, M, tok_total, K);
        else if (x_dtype == B200Q_DT_F16) gemm_xprep_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const __half*>(X), xp, M, tok_total, K);
        else gemm_xprep_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(X), xp, M, tok_total, K);
        B200Q_CUDA_TRY(cudaGetLastError());
    }
    const int ysz = y_dtype == B200Q_DT_F32 ? 4 : 2;
    for (int t0 = 0; t0 < M; t0 += kMaxTokens) {
        GemmParams p = {};
        p.W = static_cast<const uint8_t*>(W);
        p.Xp = static_cast<const uint8_t*>(ws) + (size_t)t0 * 128u;
        p.bias = bias;
        p.Y = static_cast<char*>(Y) + (size_t)t0 * N * ysz;
        p.status = status;
        p.tokens = M - t0 < kMaxTokens ? M - t0 : kMaxTokens;
        p.tok_pad = round_up16(p.tokens);
        p.xp_tok_stride = tok_total;
        p.N = N;
        p.K = K;
        p.row_bytes = (K / b200q_block_elems(fmt)) * b200q_block_bytes(fmt);
        p.bias_dtype = x_dtype;
        p.y_dtype = y_dtype;
        p.stage_bytes = kGemmRows * 128 + p.tok_pad * 128;
        int ns = (int)((227u * 1024u - 3072u) / (unsigned)p.stage_bytes);
        p.n_stages = ns > kGemmMaxStages ? kGemmMaxStages : ns;
        if (p.n_stages < 2) return fail(B200Q_ERR_UNSUPPORTED, "gemm: stage of %d bytes does not fit twice", p.stage_bytes);
        const size_t smem = (size_t)p.n_stages * p.stage_bytes + 1024;
        int rc;
        if (fmt == kQ4_K) rc = launch_gemm_fmt<kQ4_K>(p, smem, st);
        else if (fmt == kQ6_K) rc = launch_gemm_fmt<kQ6_K>(p, smem, st);
        else rc = launch_gemm_fmt<kQ8_0>(p, smem, st);
        if (rc) return rc;
    }
    return B200Q_OK;
}

}  // namespace b200q

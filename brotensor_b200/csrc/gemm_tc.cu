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
#include "gemm_common.cuh"

namespace b200q {

constexpr int kGemmThreads = 192;        // warp 0: B loader, warp 1: MMA issuer + TMEM, warps 2..5: A producers / epilogue

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

int launch_gemm_pair_pass(int fmt, const void* W, const uint8_t* Xp, int tok_stride, const void* bias, int bias_dtype,
                          void* Y, int y_dtype, int tokens, int N, int K, int n_split, float* ypart, int* status, cudaStream_t st);
// non-zero: passes run on CTA pairs (gemm_tc2.cu, the default); 0: one CTA per 128 weight rows
// (this file; kept as the reference the pair kernel is compared with bit for bit)
static int g_gemm_pair = -1;
void gemm_set_pair(int v) { g_gemm_pair = v < 0 ? -1 : (v ? 1 : 0); }
int gemm_get_pair() { return g_gemm_pair; }

static bool gemm_tc_takes(int fmt, const void* W, int M, int K) {
    if (M <= 8) return false;                 // small batches stream the weight through the decode GEMV
    if (K % 256 != 0) return false;
    if ((reinterpret_cast<uintptr_t>(W) & 15) != 0) return false;  // the producers load aligned words / 16-byte blocks
    if (fmt == kQ6_KP) return K % kQ6RunElems == 0;
    return fmt == kQ4_K || fmt == kQ6_K || fmt == kQ8_0;
}

// Split K. A pass runs one CTA pair per 256 weight rows: 4096 rows are 16 pairs on 32 of the 148 SMs.
// With at most half of the SMs busy the k-blocks of a row tile are split over up to eight pairs
// (equal shares, whole 256-element blocks, at least eight k-blocks each); the partial sums go through
// the workspace and are added in a fixed order. 1 = no split.
static int g_gemm_split = 1;
void gemm_set_split(int v) { g_gemm_split = v ? 1 : 0; }
int gemm_get_split() { return g_gemm_split; }
static int gemm_split_factor(int fmt, int N, int K) {
    if (!g_gemm_split || g_gemm_pair == 0 || N % 4 != 0) return 1;
    const int pairs = ((N + kGemmRows - 1) / kGemmRows + 1) / 2, n_kb = K / kBK;
    if (pairs > 37) return 1;
    int s = 74 / pairs;
    if (s > 8) s = 8;
    while (s > 1 && (n_kb % (4 * s) != 0 || n_kb / s < 8)) --s;
    return s;
}
static size_t gemm_xp_bytes(int M, int K) { return ((size_t)(K / kBK) * (size_t)round_up16(M) * 128u + 255u) & ~(size_t)255u; }

// What a call needs at least (the activation image) and what it asks for (with room for the partial
// sums of a split K; given less, the call runs unsplit).
size_t gemm_tc_workspace_min_bytes(int fmt, int x_dtype, int M, int N, int K) {
    (void)x_dtype; (void)N;
    if (!gemm_tc_takes(fmt, nullptr, M, K)) return 0;
    return gemm_xp_bytes(M, K);
}
size_t gemm_tc_workspace_bytes(int fmt, int x_dtype, int M, int N, int K) {
    (void)x_dtype;
    if (!gemm_tc_takes(fmt, nullptr, M, K)) return 0;
    const int s = gemm_split_factor(fmt, N, K);
    return gemm_xp_bytes(M, K) + (s > 1 ? (size_t)s * (size_t)(M < kMaxTokens ? M : kMaxTokens) * N * sizeof(float) : 0);
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
    const size_t need = gemm_tc_workspace_min_bytes(fmt, x_dtype, M, N, K);
    // (the reduction kernel moves four neighbouring outputs at a time: Y and an FP32 bias must be aligned for that)
    const bool quads_ok = (reinterpret_cast<uintptr_t>(Y) & (y_dtype == B200Q_DT_F32 ? 15 : 3)) == 0 &&
                          (!bias || x_dtype != B200Q_DT_F32 || (reinterpret_cast<uintptr_t>(bias) & 15) == 0);
    const int n_split = ws && quads_ok && ws_bytes >= gemm_tc_workspace_bytes(fmt, x_dtype, M, N, K) ? gemm_split_factor(fmt, N, K) : 1;
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
        if (g_gemm_pair != 0) {
            const int tokens = M - t0 < kMaxTokens ? M - t0 : kMaxTokens;
            if (int rc = launch_gemm_pair_pass(fmt, W, static_cast<const uint8_t*>(ws) + (size_t)t0 * 128u, tok_total, bias, x_dtype,
                                               static_cast<char*>(Y) + (size_t)t0 * N * ysz, y_dtype, tokens, N, K, n_split,
                                               reinterpret_cast<float*>(static_cast<char*>(ws) + gemm_xp_bytes(M, K)), status, st))
                return rc;
            continue;
        }
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
        else if (fmt == kQ6_KP) rc = launch_gemm_fmt<kQ6_KP>(p, smem, st);
        else rc = launch_gemm_fmt<kQ8_0>(p, smem, st);
        if (rc) return rc;
    }
    return B200Q_OK;
}

}  // namespace b200q

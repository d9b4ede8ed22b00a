// Block decode kernels: quantized rows -> FP16 / BF16 / FP32.
//
// One thread decodes eight consecutive elements (one 16-byte FP16 store), so a
// warp writes 512 contiguous bytes; the grid is a flat 1-D sweep over all
// eight-element groups, which has no 65535-row limit. Behaviour follows
// brotensor's dequant_q4k_to_fp16 (src/cuda/q4k.cu:53-96, 297-324),
// dequant_q6k_to_fp16 (q6k.cu:46-76) and dequant_q8_0_to_fp16 (q8_0.cu:40-54):
// FP32 decode, then round-to-nearest-even to the output type.
#include "common.cuh"

namespace b200q {

template <int FMT, typename OT>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ W, OT* __restrict__ out,
                                                      long long total_units, int units_per_row, int row_bytes) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x; id < total_units; id += stride) {
        const long long r = id / units_per_row;
        const int u = (int)(id - r * units_per_row);
        float w[8];
        decode8<FMT>(W + (size_t)r * row_bytes, u, w);
        OT* o = out + (size_t)id * 8;
        if constexpr (sizeof(OT) == 2) {
            union {
                OT h[8];
                uint4 v;
            } pk;
#pragma unroll
            for (int k = 0; k < 8; ++k) pk.h[k] = from_f32<OT>(w[k]);
            *reinterpret_cast<uint4*>(o) = pk.v;
        } else {
            reinterpret_cast<float4*>(o)[0] = make_float4(w[0], w[1], w[2], w[3]);
            reinterpret_cast<float4*>(o)[1] = make_float4(w[4], w[5], w[6], w[7]);
        }
    }
}

// Q4_K -> FP16, one thread per 32-element sub-block: the block header (one 16-byte load, shared
// through L1 by the block's eight threads), the 32 quant bytes of the sub-block's group, then
// 64 contiguous output bytes; a warp writes 2 KB in a row. The value is the same exact FP32
// number as the generic path's (d * sc and dmin * m are exact, one fused rounding), rounded
// once to FP16. Needs 16-byte aligned rows. (One thread per eight elements with fully coalesced
// stores was measured too and is slower: it repeats the scale decode four times as often.)
__device__ __forceinline__ uint32_t dq_pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__global__ void __launch_bounds__(256) dequant_q4k_f16_kernel(const uint8_t* __restrict__ W, __half* __restrict__ out,
                                                              long long total_sub, int sub_per_row, int row_bytes) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x; id < total_sub; id += stride) {
        const long long r = id / sub_per_row;
        const int sidx = (int)(id - r * sub_per_row);      // sub-block along the row
        const int b = sidx >> 3, t = sidx & 7, j = t >> 1, hi = t & 1;
        const uint4* blk = reinterpret_cast<const uint4*>(W + (size_t)r * row_bytes + (size_t)b * 144);
        const uint4 h = __ldg(blk);
        const uint4 qa = __ldg(blk + 1 + 2 * j), qb = __ldg(blk + 2 + 2 * j);
        uint32_t sc, m;
        if (t < 4) {
            sc = (h.y >> (8 * t)) & 63u;
            m = (h.z >> (8 * t)) & 63u;
        } else {
            const int J = t - 4;
            sc = ((h.w >> (8 * J)) & 0xFu) | (((h.y >> (8 * J + 6)) & 3u) << 4);
            m = ((h.w >> (8 * J + 4)) & 0xFu) | (((h.z >> (8 * J + 6)) & 3u) << 4);
        }
        const float ds = h2f(h.x & 0xFFFFu) * (float)sc, dm = h2f(h.x >> 16) * (float)m;
        const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
        const uint32_t sh = 4u * (uint32_t)hi;
        uint4* o = reinterpret_cast<uint4*>(out + (size_t)id * 32);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t v[4];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const uint32_t nib = (w[2 * c + k] >> sh) & 0x0F0F0F0Fu;
                float f[4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    f[i] = fmaf(ds, __uint_as_float(__byte_perm(nib, 0x4B000000u, 0x7440 | i)) - 8388608.0f, -dm);
                v[2 * k] = dq_pack_h2(f[0], f[1]);
                v[2 * k + 1] = dq_pack_h2(f[2], f[3]);
            }
            o[c] = make_uint4(v[0], v[1], v[2], v[3]);
        }
    }
}

template <int FMT>
static int launch_dequant_fmt(const void* W, void* out, int out_dtype, int64_t rows, int K, cudaStream_t st) {
    const int upr = K / 8;
    const long long total = (long long)rows * upr;
    const int row_bytes = (K / Blk<FMT>::elems) * Blk<FMT>::bytes;
    long long blocks = (total + 255) / 256;
    const long long cap = 148LL * 8 * 16;
    if (blocks > cap) blocks = cap;
    const uint8_t* w = static_cast<const uint8_t*>(W);
    if constexpr (FMT == kQ4_K) {
        if (out_dtype == B200Q_DT_F16 && (reinterpret_cast<uintptr_t>(W) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
            const long long total_sub = (long long)rows * (K / 32);
            long long nb = (total_sub + 255) / 256;
            if (nb > cap) nb = cap;
            dequant_q4k_f16_kernel<<<(unsigned)nb, 256, 0, st>>>(w, (__half*)out, total_sub, K / 32, row_bytes);
            B200Q_CUDA_TRY(cudaGetLastError());
            return B200Q_OK;
        }
    }
    switch (out_dtype) {
        case B200Q_DT_F16:
            dequant_kernel<FMT, __half><<<(unsigned)blocks, 256, 0, st>>>(w, (__half*)out, total, upr, row_bytes);
            break;
        case B200Q_DT_BF16:
            dequant_kernel<FMT, __nv_bfloat16>
                <<<(unsigned)blocks, 256, 0, st>>>(w, (__nv_bfloat16*)out, total, upr, row_bytes);
            break;
        case B200Q_DT_F32:
            dequant_kernel<FMT, float><<<(unsigned)blocks, 256, 0, st>>>(w, (float*)out, total, upr, row_bytes);
            break;
        default:
            return fail(B200Q_ERR_BAD_ARG, "dequant: unknown output dtype %d", out_dtype);
    }
    B200Q_CUDA_TRY(cudaGetLastError());
    return B200Q_OK;
}

int launch_dequant(int fmt, const void* W, void* out, int out_dtype, int64_t rows, int K, cudaStream_t st) {
    switch (fmt) {
        case kQ4_K: return launch_dequant_fmt<kQ4_K>(W, out, out_dtype, rows, K, st);
        case kQ6_K: return launch_dequant_fmt<kQ6_K>(W, out, out_dtype, rows, K, st);
        case kQ8_0: return launch_dequant_fmt<kQ8_0>(W, out, out_dtype, rows, K, st);
    }
    return fail(B200Q_ERR_BAD_ARG, "dequant: unknown block format %d", fmt);
}

}  // namespace b200q

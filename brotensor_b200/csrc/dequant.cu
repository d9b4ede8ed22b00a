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

// Q4_K -> FP16, one thread per eight positions of two neighbouring 64-element groups: the block
// header (one 16-byte load, shared through L1 by the block's eight threads), 8 quant bytes of each
// group, and 32 values - eight consecutive ones in each of four sub-blocks - so four 16-byte stores,
// with neighbouring threads writing neighbouring 16-byte pieces. The four sub-blocks' 6-bit scales
// and mins are unpacked four at a time. The value is the same exact FP32 number as the generic
// path's (d * sc and dmin * m are exact, one fused rounding), rounded once to FP16. Needs 16-byte
// aligned rows. (One thread per sub-block with 64 contiguous output bytes per thread: 11.1 us for
// 4096 x 4096 against this form's figure in the benchmark's extras.)
__device__ __forceinline__ uint32_t dq_pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__global__ void __launch_bounds__(256) dequant_q4k_f16_kernel(const uint8_t* __restrict__ W, __half* __restrict__ out,
                                                              long long total_units, int units_per_row, int row_bytes, int K) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x; id < total_units; id += stride) {
        const long long r = id / units_per_row;
        const int u = (int)(id - r * units_per_row);  // eight units per block
        const int b = u >> 3, jp = (u >> 2) & 1, p = u & 3;
        const uint8_t* blk = W + (size_t)r * row_bytes + (size_t)b * 144;
        const uint4 h = __ldg(reinterpret_cast<const uint4*>(blk));
        const uint2 g0 = __ldg(reinterpret_cast<const uint2*>(blk + 16 + 64 * jp + 8 * p));
        const uint2 g1 = __ldg(reinterpret_cast<const uint2*>(blk + 48 + 64 * jp + 8 * p));
        // scales / mins of sub-blocks 4 jp .. 4 jp + 3, one per byte
        const uint32_t scw = jp ? ((h.w & 0x0f0f0f0fu) | ((h.y >> 2) & 0x30303030u)) : (h.y & 0x3f3f3f3fu);
        const uint32_t mw = jp ? (((h.w >> 4) & 0x0f0f0f0fu) | ((h.z >> 2) & 0x30303030u)) : (h.z & 0x3f3f3f3fu);
        const float d = h2f(h.x & 0xFFFFu), dmin = h2f(h.x >> 16);
        __half* o = out + (size_t)r * K + (size_t)b * 256 + 128 * jp + 8 * p;
#pragma unroll
        for (int q = 0; q < 4; ++q) {  // sub-block 4 jp + q: low (q even) or high (q odd) nibbles of group 2 jp + q / 2
            const float ds = d * (float)((scw >> (8 * q)) & 0xFFu), dm = dmin * (float)((mw >> (8 * q)) & 0xFFu);
            const uint2 g = q < 2 ? g0 : g1;
            const uint32_t w[2] = {g.x, g.y};
            uint32_t v[4];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const uint32_t nib = ((q & 1) ? (w[k] >> 4) : w[k]) & 0x0F0F0F0Fu;
                float f[4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    f[i] = fmaf(ds, __uint_as_float(__byte_perm(nib, 0x4B000000u, 0x7440 | i)) - 8388608.0f, -dm);
                v[2 * k] = dq_pack_h2(f[0], f[1]);
                v[2 * k + 1] = dq_pack_h2(f[2], f[3]);
            }
            *reinterpret_cast<uint4*>(o + 32 * q) = make_uint4(v[0], v[1], v[2], v[3]);
        }
    }
}

// Q6_K -> FP16, one thread per eight positions l0..l0+7 of one 128-element half block: its 8 low-nibble
// bytes for the quarters 0/2 and 1/3 and its 8 high-bit bytes give 32 values - eight consecutive ones in
// each of the half's four 32-element quarters - so four 16-byte stores, and the loads and the scale
// work of the generic path are shared by four times as many outputs. Blocks are 2-byte aligned only;
// all loads are 16-bit pairs. d * sc * (q - 32) is exact in FP32 (11 + 7 + 6 bits), one rounding to FP16.
template <bool RUNS>  // RUNS: the layout regrouped by field in runs of eight blocks (16-byte aligned fields)
__global__ void __launch_bounds__(256) dequant_q6k_f16_kernel(const uint8_t* __restrict__ W, __half* __restrict__ out,
                                                              long long total_units, int units_per_row, int row_bytes, int K) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x; id < total_units; id += stride) {
        const long long r = id / units_per_row;
        const int u = (int)(id - r * units_per_row);  // eight units per block
        const int b = u >> 3, n = (u >> 2) & 1, l0 = (u & 3) * 8;
        uint32_t a[2][2], h[2];
        const uint8_t* sp;  // the half's eight sub-block scales; quarter q of positions l0.. uses scale (l0 >> 4) + 2 q
        float d;
        if constexpr (RUNS) {
            const uint8_t* run = W + (size_t)r * row_bytes + (size_t)(b >> 3) * kQ6RunBytes;
            const int s = b & 7;
            const uint2 a0 = __ldg(reinterpret_cast<const uint2*>(run + s * 128 + n * 64 + l0));
            const uint2 a1 = __ldg(reinterpret_cast<const uint2*>(run + s * 128 + n * 64 + 32 + l0));
            const uint2 hh = __ldg(reinterpret_cast<const uint2*>(run + 1024 + s * 64 + n * 32 + l0));
            a[0][0] = a0.x; a[0][1] = a0.y; a[1][0] = a1.x; a[1][1] = a1.y;
            h[0] = hh.x; h[1] = hh.y;
            sp = run + 1536 + s * 16 + n * 8 + (l0 >> 4);
            d = h2f(ld_nc_u16(run + 1664 + 2 * s));
        } else {
            const uint8_t* blk = W + (size_t)r * row_bytes + (size_t)b * 210;
            const uint8_t* ql = blk + n * 64 + l0;
            const uint8_t* qh = blk + 128 + n * 32 + l0;
            a[0][0] = ld_nc_u32_a2(ql); a[0][1] = ld_nc_u32_a2(ql + 4);
            a[1][0] = ld_nc_u32_a2(ql + 32); a[1][1] = ld_nc_u32_a2(ql + 36);
            h[0] = ld_nc_u32_a2(qh); h[1] = ld_nc_u32_a2(qh + 4);
            sp = blk + 192 + n * 8 + (l0 >> 4);
            d = h2f(ld_nc_u16(blk + 208));
        }
        __half* o = out + (size_t)r * K + (size_t)b * 256 + n * 128 + l0;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float ds = d * (float)(int)(signed char)__ldg(sp + 2 * q);
            uint32_t v[4];
#pragma unroll
            for (int w = 0; w < 2; ++w) {
                const uint32_t nib = (q < 2 ? a[q & 1][w] : (a[q & 1][w] >> 4)) & 0x0F0F0F0Fu;
                const uint32_t hb = ((h[w] >> (2 * q)) & 0x03030303u) << 4;
                const uint32_t six = nib | hb;  // four 6-bit values, one per byte
                float f[4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    f[i] = ds * (__uint_as_float(__byte_perm(six, 0x4B000000u, 0x7440 | i)) - 8388640.0f);  // byte - 32
                v[2 * w] = dq_pack_h2(f[0], f[1]);
                v[2 * w + 1] = dq_pack_h2(f[2], f[3]);
            }
            *reinterpret_cast<uint4*>(o + 32 * q) = make_uint4(v[0], v[1], v[2], v[3]);
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
            const long long total_units = (long long)rows * (K / 32);
            long long nb = (total_units + 255) / 256;
            if (nb > cap) nb = cap;
            dequant_q4k_f16_kernel<<<(unsigned)nb, 256, 0, st>>>(w, (__half*)out, total_units, K / 32, row_bytes, K);
            B200Q_CUDA_TRY(cudaGetLastError());
            return B200Q_OK;
        }
    }
    if constexpr (FMT == kQ6_K || FMT == kQ6_KP) {
        if (out_dtype == B200Q_DT_F16 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 && K % 8 == 0) {
            const long long total_units = (long long)rows * (K / 32);
            long long nb = (total_units + 255) / 256;
            if (nb > cap) nb = cap;
            dequant_q6k_f16_kernel<FMT == kQ6_KP><<<(unsigned)nb, 256, 0, st>>>(w, (__half*)out, total_units, K / 32, row_bytes, K);
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
        case kQ6_KP: return launch_dequant_fmt<kQ6_KP>(W, out, out_dtype, rows, K, st);
        case kQ8_0: return launch_dequant_fmt<kQ8_0>(W, out, out_dtype, rows, K, st);
        case kQ4_0: return launch_dequant_fmt<kQ4_0>(W, out, out_dtype, rows, K, st);
        case kQ5_K: return launch_dequant_fmt<kQ5_K>(W, out, out_dtype, rows, K, st);
    }
    return fail(B200Q_ERR_BAD_ARG, "dequant: unknown block format %d", fmt);
}

// Row gather with decode (a quantized embedding table): the dequant kernel with the row taken from
// an index vector. One thread decodes eight consecutive elements of one gathered row; an index
// outside the table writes zeros and reads nothing.
template <int FMT, typename OT>
__global__ void __launch_bounds__(256) gather_kernel(const uint8_t* __restrict__ W, const int32_t* __restrict__ idx, OT* __restrict__ out,
                                                     long long total_units, int units_per_row, int row_bytes, long long rows) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x; id < total_units; id += stride) {
        const long long b = id / units_per_row;
        const int u = (int)(id - b * units_per_row);
        const long long r = (long long)__ldg(idx + b);
        float w[8];
        if (r >= 0 && r < rows) {
            decode8<FMT>(W + (size_t)r * row_bytes, u, w);
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) w[k] = 0.f;
        }
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

template <int FMT>
static int launch_gather_fmt(const void* W, const int32_t* idx, void* out, int out_dtype, int B, int64_t rows, int K, cudaStream_t st) {
    const int upr = K / 8;
    const long long total = (long long)B * upr;
    const int row_bytes = (K / Blk<FMT>::elems) * Blk<FMT>::bytes;
    long long blocks = (total + 255) / 256;
    const long long cap = 148LL * 8 * 16;
    if (blocks > cap) blocks = cap;
    const uint8_t* w = static_cast<const uint8_t*>(W);
    switch (out_dtype) {
        case B200Q_DT_F16: gather_kernel<FMT, __half><<<(unsigned)blocks, 256, 0, st>>>(w, idx, (__half*)out, total, upr, row_bytes, rows); break;
        case B200Q_DT_BF16: gather_kernel<FMT, __nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(w, idx, (__nv_bfloat16*)out, total, upr, row_bytes, rows); break;
        case B200Q_DT_F32: gather_kernel<FMT, float><<<(unsigned)blocks, 256, 0, st>>>(w, idx, (float*)out, total, upr, row_bytes, rows); break;
        default: return fail(B200Q_ERR_BAD_ARG, "embedding_gather: unknown output dtype %d", out_dtype);
    }
    B200Q_CUDA_TRY(cudaGetLastError());
    return B200Q_OK;
}

int launch_gather(int fmt, const void* W, const int32_t* idx, void* out, int out_dtype, int B, int64_t rows, int K, cudaStream_t st) {
    switch (fmt) {
        case kQ4_K: return launch_gather_fmt<kQ4_K>(W, idx, out, out_dtype, B, rows, K, st);
        case kQ6_K: return launch_gather_fmt<kQ6_K>(W, idx, out, out_dtype, B, rows, K, st);
        case kQ6_KP: return launch_gather_fmt<kQ6_KP>(W, idx, out, out_dtype, B, rows, K, st);
        case kQ8_0: return launch_gather_fmt<kQ8_0>(W, idx, out, out_dtype, B, rows, K, st);
        case kQ4_0: return launch_gather_fmt<kQ4_0>(W, idx, out, out_dtype, B, rows, K, st);
        case kQ5_K: return launch_gather_fmt<kQ5_K>(W, idx, out, out_dtype, B, rows, K, st);
    }
    return fail(B200Q_ERR_BAD_ARG, "embedding_gather: unknown block format %d", fmt);
}

}  // namespace b200q

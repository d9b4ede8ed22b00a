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

template <int FMT>
static int launch_dequant_fmt(const void* W, void* out, int out_dtype, int64_t rows, int K, cudaStream_t st) {
    const int upr = K / 8;
    const long long total = (long long)rows * upr;
    const int row_bytes = (K / Blk<FMT>::elems) * Blk<FMT>::bytes;
    long long blocks = (total + 255) / 256;
    const long long cap = 148LL * 8 * 16;
    if (blocks > cap) blocks = cap;
    const uint8_t* w = static_cast<const uint8_t*>(W);
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

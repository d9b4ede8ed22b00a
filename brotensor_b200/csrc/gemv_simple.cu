// Plain-load decode GEMV: one warp per output row, every lane decodes groups of
// eight consecutive weights straight from global memory and multiplies them with
// the activations in FP32. It has no alignment or shape requirements beyond the
// block size, so it is the path for shapes the streaming kernel does not take
// (rows whose byte length is not a multiple of 16, oversized activations), and
// the independent cross-check for it in the tests.
// Same contract as brotensor's linear_q4k_fp16_gemv_kernel and siblings
// (src/cuda/q4k.cu:159-224, q6k.cu:117-176, q8_0.cu:75-138), extended to
// 1..8 activation rows per pass and FP32 / BF16 activations.
#include "common.cuh"

namespace b200q {

template <typename XT>
__device__ __forceinline__ void load_x8(const XT* __restrict__ x, float v[8]) {
    if constexpr (sizeof(XT) == 4) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(x));
        const float4 b = __ldg(reinterpret_cast<const float4*>(x) + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        union {
            uint4 q;
            XT h[8];
        } pk;
        pk.q = __ldg(reinterpret_cast<const uint4*>(x));
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = to_f32<XT>(pk.h[k]);
    }
}

constexpr int kSimpleWarps = 4;

template <int FMT, typename XT, typename YT, int MT>
__global__ void __launch_bounds__(kSimpleWarps * 32)
    gemv_simple_kernel(const uint8_t* __restrict__ W, const XT* __restrict__ X, const XT* __restrict__ bias,
                       YT* __restrict__ Y, int M, int N, int K, int row_bytes) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * kSimpleWarps + warp;
    if (n >= N) return;
    const uint8_t* row = W + (size_t)n * row_bytes;
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;
    const int units = K >> 3;
    for (int u = lane; u < units; u += 32) {
        float w[8];
        decode8<FMT>(row, u, w);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < M) {
                float xv[8];
                load_x8<XT>(X + (size_t)m * K + (size_t)u * 8, xv);
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[m] = fmaf(w[k], xv[k], acc[m]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
    }
    if (lane == 0) {
        const float b = bias ? to_f32<XT>(bias[n]) : 0.f;
#pragma unroll
        for (int m = 0; m < MT; ++m)
            if (m < M) Y[(size_t)m * N + n] = from_f32<YT>(acc[m] + b);
    }
}

template <int FMT, typename XT, typename YT>
static int launch_simple_t(const void* W, const void* X, const void* bias, void* Y, int M, int N, int K,
                           cudaStream_t st) {
    const int row_bytes = (K / Blk<FMT>::elems) * Blk<FMT>::bytes;
    const unsigned grid = (unsigned)((N + kSimpleWarps - 1) / kSimpleWarps);
    const uint8_t* w = static_cast<const uint8_t*>(W);
    const XT* x = static_cast<const XT*>(X);
    const XT* b = static_cast<const XT*>(bias);
    YT* y = static_cast<YT*>(Y);
    if (M == 1) gemv_simple_kernel<FMT, XT, YT, 1><<<grid, kSimpleWarps * 32, 0, st>>>(w, x, b, y, M, N, K, row_bytes);
    else if (M == 2) gemv_simple_kernel<FMT, XT, YT, 2><<<grid, kSimpleWarps * 32, 0, st>>>(w, x, b, y, M, N, K, row_bytes);
    else if (M <= 4) gemv_simple_kernel<FMT, XT, YT, 4><<<grid, kSimpleWarps * 32, 0, st>>>(w, x, b, y, M, N, K, row_bytes);
    else gemv_simple_kernel<FMT, XT, YT, 8><<<grid, kSimpleWarps * 32, 0, st>>>(w, x, b, y, M, N, K, row_bytes);
    B200Q_CUDA_TRY(cudaGetLastError());
    return B200Q_OK;
}

template <int FMT, typename XT>
static int launch_simple_x(const void* W, const void* X, const void* bias, void* Y, int y_dtype, int M, int N, int K,
                           cudaStream_t st) {
    switch (y_dtype) {
        case B200Q_DT_F32: return launch_simple_t<FMT, XT, float>(W, X, bias, Y, M, N, K, st);
        case B200Q_DT_F16: return launch_simple_t<FMT, XT, __half>(W, X, bias, Y, M, N, K, st);
        case B200Q_DT_BF16: return launch_simple_t<FMT, XT, __nv_bfloat16>(W, X, bias, Y, M, N, K, st);
    }
    return fail(B200Q_ERR_BAD_ARG, "gemv: unknown output dtype %d", y_dtype);
}

template <int FMT>
static int launch_simple_f(const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype, int M,
                           int N, int K, cudaStream_t st) {
    switch (x_dtype) {
        case B200Q_DT_F32: return launch_simple_x<FMT, float>(W, X, bias, Y, y_dtype, M, N, K, st);
        case B200Q_DT_F16: return launch_simple_x<FMT, __half>(W, X, bias, Y, y_dtype, M, N, K, st);
        case B200Q_DT_BF16: return launch_simple_x<FMT, __nv_bfloat16>(W, X, bias, Y, y_dtype, M, N, K, st);
    }
    return fail(B200Q_ERR_BAD_ARG, "gemv: unknown activation dtype %d", x_dtype);
}

int launch_gemv_simple(int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype,
                       int M, int N, int K, cudaStream_t st) {
    switch (fmt) {
        case kQ4_K: return launch_simple_f<kQ4_K>(W, X, x_dtype, bias, Y, y_dtype, M, N, K, st);
        case kQ6_K: return launch_simple_f<kQ6_K>(W, X, x_dtype, bias, Y, y_dtype, M, N, K, st);
        case kQ6_KP: return launch_simple_f<kQ6_KP>(W, X, x_dtype, bias, Y, y_dtype, M, N, K, st);
        case kQ8_0: return launch_simple_f<kQ8_0>(W, X, x_dtype, bias, Y, y_dtype, M, N, K, st);
        case kQ4_0: return launch_simple_f<kQ4_0>(W, X, x_dtype, bias, Y, y_dtype, M, N, K, st);
        case kQ5_K: return launch_simple_f<kQ5_K>(W, X, x_dtype, bias, Y, y_dtype, M, N, K, st);
    }
    return fail(B200Q_ERR_BAD_ARG, "gemv: unknown block format %d", fmt);
}

}  // namespace b200q

// C entry points over brotensor's own PUBLIC quant ops, for the same-box comparator (oracle/_ref/
// libref_cuda.so: brotensor's core plus its stock CUDA quant kernels compiled for sm_100a). The
// benchmark wraps device buffers it already holds into non-owning brotensor Tensors and calls the ops
// exactly as a brotensor user would; the stream is brotensor's own thread-local current stream.
// TEST / BENCHMARK INFRASTRUCTURE: nothing in the product links this.
#include <brotensor/ops.h>
#include <brotensor/runtime.h>
#include <brotensor/tensor.h>

#include <cstdio>
#include <exception>
#include <string>

namespace brotensor::detail::cuda {
void cuda_set_stream(void* stream, int dev);  // src/cuda/runtime.cu:66-74
}

using brotensor::Device;
using brotensor::Dtype;
using brotensor::Tensor;

static thread_local std::string g_err;

template <typename F>
static int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return 1;
    }
}

extern "C" {

const char* refcuda_last_error() { return g_err.c_str(); }

// 1 when brotensor's CUDA backend registered (a device is present), else 0.
int refcuda_init() {
    int ok = 0;
    guarded([&] {
        brotensor::init();
        ok = brotensor::is_available(Device::CUDA) ? 1 : 0;
    });
    return ok;
}

void refcuda_set_stream(void* stream) { brotensor::detail::cuda::cuda_set_stream(stream, -1); }

// fmt: brotensor's Dtype tag (14 Q8_0, 22 Q4_K, 24 Q6_K). X, Y: FP16 device buffers, X (B, K), Y (B, N).
// B == 1 calls linear_forward_*_fp16, B > 1 linear_forward_batched_*_fp16.
int refcuda_linear(int fmt, void* W, void* X, void* Y, int B, int N, int K) {
    return guarded([&] {
        const Dtype dt = static_cast<Dtype>(fmt);
        Tensor w = Tensor::view(Device::CUDA, W, N, K, dt);
        if (B == 1) {
            Tensor x = Tensor::view(Device::CUDA, X, K, 1, Dtype::FP16), y = Tensor::view(Device::CUDA, Y, N, 1, Dtype::FP16);
            if (dt == Dtype::Q4_K) brotensor::linear_forward_q4k_fp16(w, nullptr, x, y);
            else if (dt == Dtype::Q6_K) brotensor::linear_forward_q6k_fp16(w, nullptr, x, y);
            else brotensor::linear_forward_q8_0_fp16(w, nullptr, x, y);
        } else {
            Tensor x = Tensor::view(Device::CUDA, X, B, K, Dtype::FP16), y = Tensor::view(Device::CUDA, Y, B, N, Dtype::FP16);
            if (dt == Dtype::Q4_K) brotensor::linear_forward_batched_q4k_fp16(w, nullptr, x, y);
            else if (dt == Dtype::Q6_K) brotensor::linear_forward_batched_q6k_fp16(w, nullptr, x, y);
            else brotensor::linear_forward_batched_q8_0_fp16(w, nullptr, x, y);
        }
    });
}

int refcuda_dequant(int fmt, void* W, void* out, int N, int K) {
    return guarded([&] {
        const Dtype dt = static_cast<Dtype>(fmt);
        Tensor w = Tensor::view(Device::CUDA, W, N, K, dt), o = Tensor::view(Device::CUDA, out, N, K, Dtype::FP16);
        if (dt == Dtype::Q4_K) brotensor::dequant_q4k_to_fp16(w, o);
        else if (dt == Dtype::Q6_K) brotensor::dequant_q6k_to_fp16(w, o);
        else brotensor::dequant_q8_0_to_fp16(w, o);
    });
}

}  // extern "C"

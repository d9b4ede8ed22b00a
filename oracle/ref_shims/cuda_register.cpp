// Stands in for brotensor's src/cuda/register.cu in the two GPU-side builds of oracle/Makefile: the
// stock file fills the CUDA table with every op of the library (forty fill functions, i.e. all of
// src/cuda), these builds need the quant-matmul path only. Same probe, same allocator table
// (src/cuda/tensor.cu), and a table that holds the nine quant slots:
//   -DREF_SLOTS   brotensor's own CUDA kernels (src/cuda/q4k.cu, q6k.cu, q8_0.cu and their WMMA files):
//                 the same-box comparator on sm_100a
//   otherwise     this repository's backend through brotensor_b200/integration/brotensor_backend.cpp:
//                 brotensor's own parity tests against the replaced slots
// TEST INFRASTRUCTURE: built into oracle/_ref only.
#include <brotensor/detail/dispatch.h>
#include <brotensor/tensor.h>

#include <cuda_runtime_api.h>

namespace brotensor::detail::cuda {
const ::brotensor::detail::AllocVTable& cuda_alloc_table();  // src/cuda/tensor.cu:271
void init_async_pool_for_device(int dev);                    // src/cuda/tensor.cu:56
#ifdef REF_SLOTS
void dequant_q4k_to_fp16(const Tensor&, Tensor&);
void linear_forward_q4k_fp16(const Tensor&, const Tensor*, const Tensor&, Tensor&);
void linear_forward_batched_q4k_fp16(const Tensor&, const Tensor*, const Tensor&, Tensor&);
void dequant_q6k_to_fp16(const Tensor&, Tensor&);
void linear_forward_q6k_fp16(const Tensor&, const Tensor*, const Tensor&, Tensor&);
void linear_forward_batched_q6k_fp16(const Tensor&, const Tensor*, const Tensor&, Tensor&);
void dequant_q8_0_to_fp16(const Tensor&, Tensor&);
void linear_forward_q8_0_fp16(const Tensor&, const Tensor*, const Tensor&, Tensor&);
void linear_forward_batched_q8_0_fp16(const Tensor&, const Tensor*, const Tensor&, Tensor&);
#endif
}  // namespace brotensor::detail::cuda

#ifndef REF_SLOTS
namespace b200_brotensor {
void fill_b200_quant_slots(brotensor::detail::OpsVTable& ops);
}
#endif

extern "C" void brotensor_probe_and_register_cuda() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) return;  // as src/cuda/register.cu:77-87
    ::brotensor::detail::set_cuda_device_count(n);
    for (int i = 0; i < n; ++i) {
        if (cudaSetDevice(i) != cudaSuccess) continue;
        brotensor::detail::cuda::init_async_pool_for_device(i);
    }
    cudaSetDevice(0);
    ::brotensor::detail::OpsVTable ops{};
#ifdef REF_SLOTS
    namespace dc = ::brotensor::detail::cuda;
    ops.dequant_q4k_to_fp16 = dc::dequant_q4k_to_fp16;
    ops.linear_forward_q4k_fp16 = dc::linear_forward_q4k_fp16;
    ops.linear_forward_batched_q4k_fp16 = dc::linear_forward_batched_q4k_fp16;
    ops.dequant_q6k_to_fp16 = dc::dequant_q6k_to_fp16;
    ops.linear_forward_q6k_fp16 = dc::linear_forward_q6k_fp16;
    ops.linear_forward_batched_q6k_fp16 = dc::linear_forward_batched_q6k_fp16;
    ops.dequant_q8_0_to_fp16 = dc::dequant_q8_0_to_fp16;
    ops.linear_forward_q8_0_fp16 = dc::linear_forward_q8_0_fp16;
    ops.linear_forward_batched_q8_0_fp16 = dc::linear_forward_batched_q8_0_fp16;
#else
    b200_brotensor::fill_b200_quant_slots(ops);
#endif
    ::brotensor::detail::register_backend(::brotensor::DeviceType::CUDA, ops, ::brotensor::detail::cuda::cuda_alloc_table());
}

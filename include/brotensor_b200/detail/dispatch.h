// Backend tables and dispatcher of the b200 host layer. Same mechanism as
// brotensor's (include/brotensor/detail/dispatch.h:24-143, src/dispatch.cpp): one
// function-pointer slot per public op whose type is the public signature, one
// allocator table per backend, device resolution from the first committed operand.
// Only the nine quant slots exist here.
#pragma once

#include <cstdint>

#include <cstddef>
#include <initializer_list>

#include "../tensor.h"

namespace brotensor_b200::detail {

using DequantFn = void (*)(const Tensor& W, Tensor& out);
using LinearFn = void (*)(const Tensor& W, const Tensor* bias, const Tensor& x, Tensor& y);
using GroupFn = void (*)(const Tensor* const* W, const Tensor* const* bias, int n, const Tensor& x, Tensor* const* y);

struct OpsVTable {
    DequantFn dequant_q4k_to_fp16 = nullptr;
    LinearFn linear_forward_q4k_fp16 = nullptr;
    LinearFn linear_forward_batched_q4k_fp16 = nullptr;
    DequantFn dequant_q8_0_to_fp16 = nullptr;
    LinearFn linear_forward_q8_0_fp16 = nullptr;
    LinearFn linear_forward_batched_q8_0_fp16 = nullptr;
    DequantFn dequant_q6k_to_fp16 = nullptr;
    LinearFn linear_forward_q6k_fp16 = nullptr;
    LinearFn linear_forward_batched_q6k_fp16 = nullptr;
    // Extension: the two commonest GGUF formats that brotensor's loader carries without ops (src/gguf.cpp:111-130).
    DequantFn dequant_q4_0_to_fp16 = nullptr;
    LinearFn linear_forward_q4_0_fp16 = nullptr;
    LinearFn linear_forward_batched_q4_0_fp16 = nullptr;
    DequantFn dequant_q5k_to_fp16 = nullptr;
    LinearFn linear_forward_q5k_fp16 = nullptr;
    LinearFn linear_forward_batched_q5k_fp16 = nullptr;
    // brotensor's embedding_lookup_forward (include/brotensor/ops/embedding.h:14-16), here for QUANTIZED tables,
    // which brotensor refuses (src/cuda/embedding.cu:150-154).
    void (*embedding_lookup_forward)(const Tensor& table, const std::int32_t* d_idx, int B, Tensor& out) = nullptr;
    // Extension, not in brotensor's table: several matrices against one activation vector.
    GroupFn linear_forward_group_fp16 = nullptr;
    // Extension: gate and up projection with the SwiGLU gate applied in the kernel's epilogue.
    void (*linear_forward_swiglu_fp16)(const Tensor& W_gate, const Tensor& W_up, const Tensor& x, Tensor& y) = nullptr;
    // Extension: the grouped op on rms_norm(x) * gamma, the normalisation folded into the launch.
    void (*linear_forward_group_rmsnorm_fp16)(const Tensor* const* W, int n, const Tensor& x, const Tensor& gamma, float eps,
                                              Tensor* const* y) = nullptr;
};

struct AllocVTable {
    void* (*alloc)(std::size_t bytes, int device_index) = nullptr;
    void (*free)(void* ptr, int device_index) = nullptr;
    void (*memcpy_h2d)(void* dst, const void* src, std::size_t n, int device_index) = nullptr;
    void (*memcpy_d2h)(void* dst, const void* src, std::size_t n, int device_index) = nullptr;
    void (*memcpy_d2d)(void* dst, const void* src, std::size_t n, int device_index) = nullptr;
    // Stream-ordered copies that return at once; `src` / `dst` on the host should be page-locked
    // (pageable memory works but makes the copy synchronous). Not in brotensor's table.
    void (*memcpy_h2d_async)(void* dst, const void* src, std::size_t n, int device_index) = nullptr;
    void (*memcpy_d2h_async)(void* dst, const void* src, std::size_t n, int device_index) = nullptr;
    void (*memcpy_peer)(void* dst, int dst_device, const void* src, int src_device, std::size_t n) = nullptr;
    void (*memset_zero)(void* dst, std::size_t n, int device_index) = nullptr;
    void (*sync)(int device_index) = nullptr;
    bool (*mem_info)(std::size_t* free_bytes, std::size_t* total_bytes, int device_index) = nullptr;
    bool (*device_name)(char* out, std::size_t cap, int device_index) = nullptr;
};

// Registering a device type twice replaces its tables.
void register_backend(DeviceType dt, const OpsVTable& ops, const AllocVTable& alloc);
const OpsVTable& ops_for(Device d);      // throws if the backend is not registered
const AllocVTable& alloc_for(Device d);  // throws if the backend is not registered
bool is_registered(Device d);
void set_cuda_device_count(int count);
int get_cuda_device_count();

// Resolve the op's device from the first operand with storage; every other operand
// with storage must agree, else std::runtime_error. Null optionals are skipped.
// Selects that CUDA device for the calling thread before returning its table.
const OpsVTable& dispatch_with_opts(const Tensor& a, std::initializer_list<const Tensor*> opts);
void adopt_output(Tensor& t, Device d);
[[noreturn]] void throw_not_implemented(const char* op_name, Device d);

}  // namespace brotensor_b200::detail

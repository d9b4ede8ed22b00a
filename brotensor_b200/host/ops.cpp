// Public op wrappers: resolve the device, refuse a null slot, pin an unsized output to
// the op's device, call the backend (brotensor src/ops.cpp:2049-2125).
#include <stdexcept>
#include <string>

#include "brotensor_b200/detail/dispatch.h"
#include "brotensor_b200/ops/quant.h"

namespace brotensor_b200 {

#define B200_DEQUANT_OP(name)                                                   \
    void name(const Tensor& W, Tensor& out) {                                   \
        const detail::OpsVTable& v = detail::dispatch_with_opts(W, {&out});     \
        const Device dev = W.data ? W.device : (out.data ? out.device : W.device); \
        if (!v.name) detail::throw_not_implemented(#name, dev);                 \
        detail::adopt_output(out, dev);                                         \
        v.name(W, out);                                                         \
    }

#define B200_LINEAR_OP(name)                                                          \
    void name(const Tensor& W, const Tensor* bias, const Tensor& x, Tensor& y) {      \
        const detail::OpsVTable& v = detail::dispatch_with_opts(W, {bias, &x, &y});   \
        Device dev = W.device;                                                        \
        if (W.data) dev = W.device;                                                   \
        else if (bias && bias->data) dev = bias->device;                              \
        else if (x.data) dev = x.device;                                              \
        else if (y.data) dev = y.device;                                              \
        if (!v.name) detail::throw_not_implemented(#name, dev);                       \
        detail::adopt_output(y, dev);                                                 \
        v.name(W, bias, x, y);                                                        \
    }

B200_DEQUANT_OP(dequant_q4k_to_fp16)
B200_LINEAR_OP(linear_forward_q4k_fp16)
B200_LINEAR_OP(linear_forward_batched_q4k_fp16)
B200_DEQUANT_OP(dequant_q8_0_to_fp16)
B200_LINEAR_OP(linear_forward_q8_0_fp16)
B200_LINEAR_OP(linear_forward_batched_q8_0_fp16)
B200_DEQUANT_OP(dequant_q6k_to_fp16)
B200_LINEAR_OP(linear_forward_q6k_fp16)
B200_LINEAR_OP(linear_forward_batched_q6k_fp16)

B200_DEQUANT_OP(dequant_q4_0_to_fp16)
B200_LINEAR_OP(linear_forward_q4_0_fp16)
B200_LINEAR_OP(linear_forward_batched_q4_0_fp16)
B200_DEQUANT_OP(dequant_q5k_to_fp16)
B200_LINEAR_OP(linear_forward_q5k_fp16)
B200_LINEAR_OP(linear_forward_batched_q5k_fp16)

void embedding_lookup_forward(const Tensor& table, const std::int32_t* d_idx, int B, Tensor& out) {
    const detail::OpsVTable& v = detail::dispatch_with_opts(table, {&out});
    if (!v.embedding_lookup_forward) detail::throw_not_implemented("embedding_lookup_forward", table.device);
    detail::adopt_output(out, table.device);
    v.embedding_lookup_forward(table, d_idx, B, out);
}

void linear_forward_group_fp16(const Tensor* const* W, const Tensor* const* bias, int n, const Tensor& x, Tensor* const* y) {
    if (n <= 0 || !W || !y || !W[0] || !y[0]) throw std::runtime_error("brotensor: linear_forward_group_fp16: no matrices");
    const detail::OpsVTable& v = detail::dispatch_with_opts(*W[0], {&x, y[0]});
    const Device dev = W[0]->device;
    if (!v.linear_forward_group_fp16) detail::throw_not_implemented("linear_forward_group_fp16", dev);
    for (int s = 0; s < n; ++s) {
        if (!W[s] || !y[s]) throw std::runtime_error("brotensor: linear_forward_group_fp16: null tensor");
        if (W[s]->device != dev) throw std::runtime_error("brotensor: linear_forward_group_fp16: matrices on different devices");
        detail::adopt_output(*y[s], dev);
    }
    v.linear_forward_group_fp16(W, bias, n, x, y);
}

void linear_forward_group_rmsnorm_fp16(const Tensor* const* W, int n, const Tensor& x, const Tensor& gamma, float eps,
                                       Tensor* const* y) {
    const char* op = "linear_forward_group_rmsnorm_fp16";
    if (n <= 0 || !W || !y || !W[0] || !y[0]) throw std::runtime_error(std::string("brotensor: ") + op + ": no matrices");
    const detail::OpsVTable& v = detail::dispatch_with_opts(*W[0], {&x, &gamma, y[0]});
    const Device dev = W[0]->device;
    if (!v.linear_forward_group_rmsnorm_fp16) detail::throw_not_implemented(op, dev);
    for (int s = 0; s < n; ++s) {
        if (!W[s] || !y[s]) throw std::runtime_error(std::string("brotensor: ") + op + ": null tensor");
        if (W[s]->device != dev) throw std::runtime_error(std::string("brotensor: ") + op + ": matrices on different devices");
        detail::adopt_output(*y[s], dev);
    }
    v.linear_forward_group_rmsnorm_fp16(W, n, x, gamma, eps, y);
}

void linear_forward_swiglu_fp16(const Tensor& W_gate, const Tensor& W_up, const Tensor& x, Tensor& y) {
    const detail::OpsVTable& v = detail::dispatch_with_opts(W_gate, {&W_up, &x, &y});
    if (!v.linear_forward_swiglu_fp16) detail::throw_not_implemented("linear_forward_swiglu_fp16", W_gate.device);
    detail::adopt_output(y, W_gate.device);
    v.linear_forward_swiglu_fp16(W_gate, W_up, x, y);
}

}  // namespace brotensor_b200

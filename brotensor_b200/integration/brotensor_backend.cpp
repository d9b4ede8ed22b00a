// The binding a brotensor maintainer adds to put the B200 quant-matmul path behind brotensor's own
// ops: nine functions with the signatures of brotensor's vtable slots (include/brotensor/detail/
// dispatch.h:24-28) that validate like the stock CUDA backend (src/cuda/q4k.cu:283-293, 326-420 and
// the q6k / q8_0 twins), resize the output and call the C-ABI of include/b200q.h on the thread's
// current stream, and install_b200_quant(), which overwrites the nine slots of the registered CUDA
// table ("registering twice replaces", detail/dispatch.h:72-76).
//
// This file compiles against brotensor's headers, not against this repository's host layer. It is
// built by oracle/Makefile (target b200_tests) together with brotensor's core sources and brotensor's
// own parity tests, which then run unmodified against the replaced slots.
#include <brotensor/detail/dispatch.h>
#include <brotensor/tensor.h>

#include <cuda_runtime_api.h>

#include <stdexcept>
#include <string>

#include "b200q.h"

namespace brotensor {
void* cuda_current_stream();  // src/cuda/runtime.cu:58-64
}

namespace b200_brotensor {

using brotensor::Dtype;
using brotensor::Tensor;

namespace {

[[noreturn]] void op_fail(const char* op, const std::string& why) { throw std::runtime_error(std::string("brotensor: ") + op + ": " + why); }

void check(int rc, const char* op) {
    if (rc == B200Q_OK) return;
    const char* msg = b200q_last_error();
    if (rc == B200Q_ERR_CUDA) throw std::runtime_error(msg);
    op_fail(op, msg && *msg ? msg : b200q_status_str(rc));
}

void validate_w(const Tensor& W, Dtype want, const char* dname, int block, const char* op) {
    if (W.dtype != want) op_fail(op, std::string("W must be Dtype::") + dname);
    if (W.cols % block != 0) op_fail(op, "W.cols must be a multiple of " + std::to_string(block));
    if (W.rows <= 0 || W.cols <= 0) op_fail(op, "W has non-positive shape");
}

void dequant(int fmt, Dtype wdt, const char* dname, int block, const char* op, const Tensor& W, Tensor& out) {
    validate_w(W, wdt, dname, block, op);
    if (out.rows != W.rows || out.cols != W.cols || out.dtype != Dtype::FP16) out.resize(W.rows, W.cols, Dtype::FP16);
    check(b200q_dequant(fmt, W.data, out.data, B200Q_DT_F16, W.rows, W.cols, brotensor::cuda_current_stream()), op);
}

void gemv(int fmt, Dtype wdt, const char* dname, int block, const char* op, const Tensor& W, const Tensor* bias, const Tensor& x,
          Tensor& y) {
    validate_w(W, wdt, dname, block, op);
    if (x.dtype != Dtype::FP16) op_fail(op, "x must be FP16");
    if (x.rows != W.cols || x.cols != 1) op_fail(op, "x shape must be (in, 1)");
    if (bias) {
        if (bias->dtype != Dtype::FP16) op_fail(op, "bias must be FP16");
        if (bias->rows != W.rows || bias->cols != 1) op_fail(op, "bias shape must be (out, 1)");
    }
    if (y.rows != W.rows || y.cols != 1 || y.dtype != Dtype::FP16) y.resize(W.rows, 1, Dtype::FP16);
    const void* b = (bias && bias->size() > 0) ? bias->data : nullptr;
    check(b200q_gemv(fmt, W.data, x.data, B200Q_DT_F16, b, y.data, B200Q_DT_F16, 1, W.rows, W.cols, brotensor::cuda_current_stream()), op);
}

void batched(int fmt, Dtype wdt, const char* dname, int block, const char* op, const Tensor& W, const Tensor* bias, const Tensor& X,
             Tensor& Y) {
    validate_w(W, wdt, dname, block, op);
    if (X.dtype != Dtype::FP16) op_fail(op, "X must be FP16");
    const int B = X.rows, K = X.cols, out = W.rows;
    if (W.cols != K) op_fail(op, "shape mismatch (W.cols != X.cols)");
    if (bias) {
        if (bias->dtype != Dtype::FP16) op_fail(op, "bias must be FP16");
        const bool ok = (bias->rows == out && bias->cols == 1) || (bias->rows == 1 && bias->cols == out);
        if (!ok) op_fail(op, "bias shape must be (out,1) or (1,out)");
    }
    if (Y.rows != B || Y.cols != out || Y.dtype != Dtype::FP16) Y.resize(B, out, Dtype::FP16);
    if (B == 0 || out == 0) return;
    const void* b = (bias && bias->size() > 0) ? bias->data : nullptr;
    cudaStream_t st = static_cast<cudaStream_t>(brotensor::cuda_current_stream());
    // workspace of the tensor-core GEMM: stream-ordered per call, as the stock ops take their scratch
    // (src/cuda/bias_act.cu:34-38)
    const size_t need = B > 8 ? b200q_gemm_workspace_bytes(fmt, B200Q_DT_F16, B, out, K) : 0;
    void* ws = nullptr;
    if (need && cudaMallocAsync(&ws, need, st) != cudaSuccess) op_fail(op, "workspace allocation failed");
    const int rc = b200q_linear(fmt, W.data, X.data, B200Q_DT_F16, b, Y.data, B200Q_DT_F16, B, out, K, ws, need, st);
    if (ws) cudaFreeAsync(ws, st);
    check(rc, op);
}

#define B200_OPS(tag, FMT, DT, DNAME, BLOCK)                                                                       \
    void dequant_##tag(const Tensor& W, Tensor& o) { dequant(FMT, DT, DNAME, BLOCK, "dequant_" #tag "_to_fp16", W, o); } \
    void gemv_##tag(const Tensor& W, const Tensor* b, const Tensor& x, Tensor& y) {                                \
        gemv(FMT, DT, DNAME, BLOCK, "linear_forward_" #tag "_fp16", W, b, x, y);                                   \
    }                                                                                                              \
    void batched_##tag(const Tensor& W, const Tensor* b, const Tensor& X, Tensor& Y) {                             \
        batched(FMT, DT, DNAME, BLOCK, "linear_forward_batched_" #tag "_fp16", W, b, X, Y);                        \
    }
B200_OPS(q4k, B200Q_FMT_Q4_K, Dtype::Q4_K, "Q4_K", 256)
B200_OPS(q6k, B200Q_FMT_Q6_K, Dtype::Q6_K, "Q6_K", 256)
B200_OPS(q8_0, B200Q_FMT_Q8_0, Dtype::Q8_0, "Q8_0", 32)

}  // namespace

// The nine slots of `ops`, whatever else it holds.
void fill_b200_quant_slots(brotensor::detail::OpsVTable& ops) {
    ops.dequant_q4k_to_fp16 = dequant_q4k;
    ops.linear_forward_q4k_fp16 = gemv_q4k;
    ops.linear_forward_batched_q4k_fp16 = batched_q4k;
    ops.dequant_q8_0_to_fp16 = dequant_q8_0;
    ops.linear_forward_q8_0_fp16 = gemv_q8_0;
    ops.linear_forward_batched_q8_0_fp16 = batched_q8_0;
    ops.dequant_q6k_to_fp16 = dequant_q6k;
    ops.linear_forward_q6k_fp16 = gemv_q6k;
    ops.linear_forward_batched_q6k_fp16 = batched_q6k;
}

// After brotensor::init(): replace the nine quant slots of the registered CUDA backend.
void install_b200_quant() {
    using namespace brotensor;
    detail::OpsVTable ops = detail::ops_for(Device::CUDA);
    fill_b200_quant_slots(ops);
    detail::register_backend(DeviceType::CUDA, ops, detail::alloc_for(Device::CUDA));
}

}  // namespace b200_brotensor

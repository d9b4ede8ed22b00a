// CUDA backend of the b200 host layer: the allocator table (stream-ordered pool
// allocation, blocking host copies, event-ordered peer copies; brotensor
// src/cuda/tensor.cu:56-187) and the nine quant ops. Each op validates like
// brotensor's (src/cuda/q4k.cu:283-293, 326-420 and the q6k / q8_0 twins), resizes the
// output, and calls the C-ABI of include/b200q.h on the thread's current stream.
#include <cuda_runtime_api.h>

#include <cstdint>
#include <mutex>
#include <stdexcept>
#include <string>

#include "b200q.h"
#include "brotensor_b200/detail/dispatch.h"
#include "brotensor_b200/runtime.h"
#include "brotensor_b200/repack.h"

namespace brotensor_b200::detail {

namespace {

[[noreturn]] void cuda_fail(cudaError_t e, const char* expr, const char* file, int line) {
    (void)cudaGetLastError();
    throw std::runtime_error("CUDA error " + std::to_string(static_cast<int>(e)) + " (" + cudaGetErrorString(e) + ") at " +
                             file + ":" + std::to_string(line) + " in `" + expr + "`");
}
#define B200_CUDA_CHECK(expr)                                        \
    do {                                                             \
        const cudaError_t e_ = (expr);                               \
        if (e_ != cudaSuccess) cuda_fail(e_, #expr, __FILE__, __LINE__); \
    } while (0)

struct DeviceGuard {
    int prev = 0;
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) B200_CUDA_CHECK(cudaSetDevice(dev));
    }
    ~DeviceGuard() { cudaSetDevice(prev); }
};

cudaStream_t cur_stream(int dev) { return static_cast<cudaStream_t>(cuda_current_stream(dev)); }

// ---- allocator table ----
void* c_alloc(std::size_t n, int dev) {
    if (!n) return nullptr;
    DeviceGuard g(dev);
    void* p = nullptr;
    B200_CUDA_CHECK(cudaMallocAsync(&p, n, cur_stream(dev)));
    return p;
}
void c_free(void* p, int dev) {
    if (!p) return;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(dev);
    if (cudaFreeAsync(p, cur_stream(dev)) != cudaSuccess) (void)cudaGetLastError();
    cudaSetDevice(prev);
}
void c_h2d(void* d, const void* s, std::size_t n, int dev) {
    DeviceGuard g(dev);
    B200_CUDA_CHECK(cudaMemcpyAsync(d, s, n, cudaMemcpyHostToDevice, cur_stream(dev)));
    B200_CUDA_CHECK(cudaStreamSynchronize(cur_stream(dev)));
}
void c_d2h(void* d, const void* s, std::size_t n, int dev) {
    DeviceGuard g(dev);
    B200_CUDA_CHECK(cudaMemcpyAsync(d, s, n, cudaMemcpyDeviceToHost, cur_stream(dev)));
    B200_CUDA_CHECK(cudaStreamSynchronize(cur_stream(dev)));
}
void c_h2d_async(void* d, const void* s, std::size_t n, int dev) {
    DeviceGuard g(dev);
    B200_CUDA_CHECK(cudaMemcpyAsync(d, s, n, cudaMemcpyHostToDevice, cur_stream(dev)));
}
void c_d2h_async(void* d, const void* s, std::size_t n, int dev) {
    DeviceGuard g(dev);
    B200_CUDA_CHECK(cudaMemcpyAsync(d, s, n, cudaMemcpyDeviceToHost, cur_stream(dev)));
}
void c_d2d(void* d, const void* s, std::size_t n, int dev) {
    DeviceGuard g(dev);
    B200_CUDA_CHECK(cudaMemcpyAsync(d, s, n, cudaMemcpyDeviceToDevice, cur_stream(dev)));
}
void c_peer(void* d, int ddev, const void* s, int sdev, std::size_t n) {
    // ordered after the source device's stream, executed on the destination's
    DeviceGuard g(sdev);
    cudaEvent_t ev;
    B200_CUDA_CHECK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    B200_CUDA_CHECK(cudaEventRecord(ev, cur_stream(sdev)));
    B200_CUDA_CHECK(cudaSetDevice(ddev));
    B200_CUDA_CHECK(cudaStreamWaitEvent(cur_stream(ddev), ev, 0));
    B200_CUDA_CHECK(cudaMemcpyPeerAsync(d, ddev, s, sdev, n, cur_stream(ddev)));
    B200_CUDA_CHECK(cudaEventDestroy(ev));
}
void c_zero(void* d, std::size_t n, int dev) {
    DeviceGuard g(dev);
    B200_CUDA_CHECK(cudaMemsetAsync(d, 0, n, cur_stream(dev)));
}
void c_sync(int dev) {
    DeviceGuard g(dev);
    B200_CUDA_CHECK(cudaDeviceSynchronize());
}
bool c_mem_info(std::size_t* f, std::size_t* t, int dev) {
    DeviceGuard g(dev);
    return cudaMemGetInfo(f, t) == cudaSuccess;
}
bool c_name(char* out, std::size_t cap, int dev) {
    cudaDeviceProp p;
    if (cudaGetDeviceProperties(&p, dev) != cudaSuccess) return false;
    std::snprintf(out, cap, "%s", p.name);
    return true;
}

// ---- the nine ops ----
[[noreturn]] void op_fail(const char* op, const std::string& why) {
    throw std::runtime_error(std::string("brotensor: ") + op + ": " + why);
}
bool act_dtype(Dtype d) { return d == Dtype::FP32 || d == Dtype::FP16 || d == Dtype::BF16; }

void check_w(const Tensor& W, Dtype want, const char* dname, int block, const char* op) {
    if (W.dtype != want) op_fail(op, std::string("W must be Dtype::") + dname);
    if (W.cols % block != 0) op_fail(op, "W.cols must be a multiple of " + std::to_string(block));
    if (W.rows <= 0 || W.cols <= 0) op_fail(op, "W has non-positive shape");
}
void check_status(int rc, const char* op) {
    if (rc == B200Q_OK) return;
    const char* msg = b200q_last_error();
    if (rc == B200Q_ERR_CUDA) throw std::runtime_error(msg);  // already "CUDA error N (...) at file:line in `expr`"
    op_fail(op, msg && *msg ? msg : b200q_status_str(rc));
}

// Workspace of the tensor-core GEMM (activations in operand layout): allocated per call from the
// stream-ordered pool on the current stream and released behind the kernel, as brotensor's ops take
// their scratch (src/cuda/bias_act.cu:34-38). That is legal inside a stream capture (the graph owns the allocation),
// safe for threads on different streams, and no pointer outlives the call that a later, larger call
// could free under a captured graph.
struct StreamScratch {
    void* p = nullptr;
    cudaStream_t st = nullptr;
    StreamScratch(std::size_t need, cudaStream_t s) : st(s) {
        if (need) B200_CUDA_CHECK(cudaMallocAsync(&p, need, st));
    }
    ~StreamScratch() {
        if (p && cudaFreeAsync(p, st) != cudaSuccess) (void)cudaGetLastError();
    }
    StreamScratch(const StreamScratch&) = delete;
    StreamScratch& operator=(const StreamScratch&) = delete;
};

// Output dtype rule shared by the ops: FP16 activations give FP16 results, always (the reference's
// contract, src/cuda/q4k.cu:345-347, 391-393: y is retyped to FP16 whatever it held); with FP32 or
// BF16 activations - which the reference does not accept - a pre-sized FP32 / FP16 / BF16 result of
// the right shape is kept and anything else becomes FP32.
bool keep_out(const Tensor& y, int rows, int cols, Dtype x_dtype) {
    if (y.rows != rows || y.cols != cols || !y.data) return false;
    return x_dtype == Dtype::FP16 ? y.dtype == Dtype::FP16 : act_dtype(y.dtype);
}

// The format code the kernels get: the raw one, or the regrouped one when W's storage is recorded as
// repacked (repack_weights).
int layout_fmt(int fmt, const Tensor& W) {
    return (fmt == B200Q_FMT_Q6_K && is_repacked(W)) ? B200Q_FMT_Q6_K_R8 : fmt;
}

void dequant_impl(int fmt, Dtype wdt, const char* dname, int block, const char* op, const Tensor& W, Tensor& out) {
    check_w(W, wdt, dname, block, op);
    // keep a pre-sized FP32 / BF16 destination, otherwise FP16 as in the reference
    const bool keep = out.rows == W.rows && out.cols == W.cols && act_dtype(out.dtype) && out.data;
    if (!keep) out.resize(W.rows, W.cols, Dtype::FP16);
    if (W.rows == 0) return;
    check_status(b200q_dequant(layout_fmt(fmt, W), W.data, out.data, static_cast<int>(out.dtype), W.rows, W.cols,
                               cuda_current_stream(W.device.index)), op);
}

void gemv_impl(int fmt, Dtype wdt, const char* dname, int block, const char* op, const Tensor& W, const Tensor* bias,
               const Tensor& x, Tensor& y) {
    check_w(W, wdt, dname, block, op);
    if (!act_dtype(x.dtype)) op_fail(op, "x must be FP16 (FP32 and BF16 are accepted as well)");
    const int out = W.rows, K = W.cols;
    if (x.rows != K || x.cols != 1) op_fail(op, "x shape must be (in, 1)");
    if (bias) {
        if (bias->dtype != x.dtype) op_fail(op, x.dtype == Dtype::FP16 ? "bias must be FP16" : "bias must have x's dtype");
        if (bias->rows != out || bias->cols != 1) op_fail(op, "bias shape must be (out, 1)");
    }
    if (!keep_out(y, out, 1, x.dtype)) y.resize(out, 1, x.dtype == Dtype::FP16 ? Dtype::FP16 : Dtype::FP32);
    if (out == 0) return;
    const void* b = (bias && bias->size() > 0) ? bias->data : nullptr;
    check_status(b200q_gemv(layout_fmt(fmt, W), W.data, x.data, static_cast<int>(x.dtype), b, y.data, static_cast<int>(y.dtype), 1, out,
                            K, cuda_current_stream(W.device.index)), op);
}

void group_impl(const Tensor* const* W, const Tensor* const* bias, int n, const Tensor& x, Tensor* const* y) {
    const char* op = "linear_forward_group_fp16";
    if (n > 4) op_fail(op, "at most four matrices per call");
    const Dtype wdt = W[0]->dtype;
    const int block = wdt == Dtype::Q8_0 ? 32 : 256;
    const char* dname = wdt == Dtype::Q4_K ? "Q4_K" : wdt == Dtype::Q6_K ? "Q6_K" : wdt == Dtype::Q8_0 ? "Q8_0" : nullptr;
    if (!dname) op_fail(op, "W must be Dtype::Q4_K, Q6_K or Q8_0");
    if (!act_dtype(x.dtype)) op_fail(op, "x must be FP16 (FP32 and BF16 are accepted as well)");
    const int K = W[0]->cols;
    if (x.rows != K || x.cols != 1) op_fail(op, "x shape must be (in, 1)");
    const void* Wp[4];
    void* Yp[4];
    const void* Bp[4];
    int Np[4];
    const Dtype ydt = x.dtype == Dtype::FP16 ? Dtype::FP16 : (y[0]->data && act_dtype(y[0]->dtype)) ? y[0]->dtype : Dtype::FP32;
    for (int s = 0; s < n; ++s) {
        check_w(*W[s], wdt, dname, block, op);
        if (W[s]->cols != K) op_fail(op, "all matrices must have the same number of columns");
        const int out = W[s]->rows;
        const Tensor* b = bias ? bias[s] : nullptr;
        if (b) {
            if (b->dtype != x.dtype) op_fail(op, x.dtype == Dtype::FP16 ? "bias must be FP16" : "bias must have x's dtype");
            if (b->rows != out || b->cols != 1) op_fail(op, "bias shape must be (out, 1)");
        }
        const bool keep = y[s]->rows == out && y[s]->cols == 1 && y[s]->dtype == ydt && y[s]->data;
        if (!keep) y[s]->resize(out, 1, ydt);
        if (is_repacked(*W[s]) != is_repacked(*W[0])) op_fail(op, "all matrices must be in the same layout (repack_weights on all or none)");
        Wp[s] = W[s]->data;
        Yp[s] = y[s]->data;
        Bp[s] = (b && b->size() > 0) ? b->data : nullptr;
        Np[s] = out;
    }
    check_status(b200q_gemv_multi(layout_fmt(static_cast<int>(wdt), *W[0]), n, Wp, Np, Yp, Bp, x.data, static_cast<int>(x.dtype), static_cast<int>(ydt), K,
                                  cuda_current_stream(W[0]->device.index)), op);
}

void group_rmsnorm_impl(const Tensor* const* W, int n, const Tensor& x, const Tensor& gamma, float eps, Tensor* const* y) {
    const char* op = "linear_forward_group_rmsnorm_fp16";
    if (n > 4) op_fail(op, "at most four matrices per call");
    const Dtype wdt = W[0]->dtype;
    const int block = wdt == Dtype::Q8_0 ? 32 : 256;
    const char* dname = wdt == Dtype::Q4_K ? "Q4_K" : wdt == Dtype::Q6_K ? "Q6_K" : wdt == Dtype::Q8_0 ? "Q8_0" : nullptr;
    if (!dname) op_fail(op, "W must be Dtype::Q4_K, Q6_K or Q8_0");
    if (!act_dtype(x.dtype)) op_fail(op, "x must be FP16 (FP32 and BF16 are accepted as well)");
    const int K = W[0]->cols;
    if (x.rows != K || x.cols != 1) op_fail(op, "x shape must be (in, 1)");
    if (gamma.dtype != x.dtype) op_fail(op, "gamma must have x's dtype");
    if (gamma.rows != K || gamma.cols != 1) op_fail(op, "gamma shape must be (in, 1)");
    if (!(eps >= 0.f)) op_fail(op, "eps must not be negative");
    const void* Wp[4];
    void* Yp[4];
    int Np[4];
    const Dtype ydt = x.dtype == Dtype::FP16 ? Dtype::FP16 : (y[0]->data && act_dtype(y[0]->dtype)) ? y[0]->dtype : Dtype::FP32;
    for (int s = 0; s < n; ++s) {
        check_w(*W[s], wdt, dname, block, op);
        if (W[s]->cols != K) op_fail(op, "all matrices must have the same number of columns");
        if (is_repacked(*W[s]) != is_repacked(*W[0])) op_fail(op, "all matrices must be in the same layout (repack_weights on all or none)");
        const int out = W[s]->rows;
        const bool keep = y[s]->rows == out && y[s]->cols == 1 && y[s]->dtype == ydt && y[s]->data;
        if (!keep) y[s]->resize(out, 1, ydt);
        Wp[s] = W[s]->data;
        Yp[s] = y[s]->data;
        Np[s] = out;
    }
    check_status(b200q_gemv_multi_rmsnorm(layout_fmt(static_cast<int>(wdt), *W[0]), n, Wp, Np, Yp, nullptr, x.data, static_cast<int>(x.dtype),
                                          gamma.data, eps, static_cast<int>(ydt), K, cuda_current_stream(W[0]->device.index)), op);
}

void swiglu_impl(const Tensor& Wg, const Tensor& Wu, const Tensor& x, Tensor& y) {
    const char* op = "linear_forward_swiglu_fp16";
    const Dtype wdt = Wg.dtype;
    const int block = wdt == Dtype::Q8_0 ? 32 : 256;
    const char* dname = wdt == Dtype::Q4_K ? "Q4_K" : wdt == Dtype::Q6_K ? "Q6_K" : wdt == Dtype::Q8_0 ? "Q8_0" : nullptr;
    if (!dname) op_fail(op, "W must be Dtype::Q4_K, Q6_K or Q8_0");
    check_w(Wg, wdt, dname, block, op);
    check_w(Wu, wdt, dname, block, op);
    if (Wu.rows != Wg.rows || Wu.cols != Wg.cols) op_fail(op, "W_gate and W_up must have the same shape");
    if (is_repacked(Wg) != is_repacked(Wu)) op_fail(op, "both matrices must be in the same layout (repack_weights on both or neither)");
    if (!act_dtype(x.dtype)) op_fail(op, "x must be FP16 (FP32 and BF16 are accepted as well)");
    const int out = Wg.rows, K = Wg.cols;
    if (x.rows != K || x.cols != 1) op_fail(op, "x shape must be (in, 1)");
    if (!keep_out(y, out, 1, x.dtype)) y.resize(out, 1, x.dtype == Dtype::FP16 ? Dtype::FP16 : Dtype::FP32);
    if (out == 0) return;
    check_status(b200q_gemv_swiglu(layout_fmt(static_cast<int>(wdt), Wg), Wg.data, Wu.data, x.data, static_cast<int>(x.dtype), y.data,
                                   static_cast<int>(y.dtype), out, K, cuda_current_stream(Wg.device.index)), op);
}

void batched_impl(int fmt, Dtype wdt, const char* dname, int block, const char* op, const Tensor& W, const Tensor* bias,
                  const Tensor& X, Tensor& Y) {
    check_w(W, wdt, dname, block, op);
    if (!act_dtype(X.dtype)) op_fail(op, "X must be FP16 (FP32 and BF16 are accepted as well)");
    const int B = X.rows, K = X.cols, out = W.rows;
    if (W.cols != K) op_fail(op, "shape mismatch (W.cols != X.cols)");
    if (bias) {
        if (bias->dtype != X.dtype) op_fail(op, X.dtype == Dtype::FP16 ? "bias must be FP16" : "bias must have X's dtype");
        const bool ok = (bias->rows == out && bias->cols == 1) || (bias->rows == 1 && bias->cols == out);
        if (!ok) op_fail(op, "bias shape must be (out,1) or (1,out)");
    }
    if (!keep_out(Y, B, out, X.dtype)) Y.resize(B, out, X.dtype == Dtype::FP16 ? Dtype::FP16 : Dtype::FP32);
    if (B == 0 || out == 0) return;
    const void* b = (bias && bias->size() > 0) ? bias->data : nullptr;
    const int dev = W.device.index;
    const int lf = layout_fmt(fmt, W);
    const std::size_t need = B > 8 ? b200q_gemm_workspace_bytes(lf, static_cast<int>(X.dtype), B, out, K) : 0;
    const StreamScratch ws(need, cur_stream(dev));
    check_status(b200q_linear(lf, W.data, X.data, static_cast<int>(X.dtype), b, Y.data, static_cast<int>(Y.dtype), B,
                              out, K, ws.p, need, cuda_current_stream(dev)), op);
}

#define B200_FMT_OPS(tag, FMT, DT, DNAME, BLOCK)                                                                 \
    void dequant_##tag(const Tensor& W, Tensor& o) { dequant_impl(FMT, DT, DNAME, BLOCK, "dequant_" #tag "_to_fp16", W, o); } \
    void gemv_##tag(const Tensor& W, const Tensor* b, const Tensor& x, Tensor& y) {                              \
        gemv_impl(FMT, DT, DNAME, BLOCK, "linear_forward_" #tag "_fp16", W, b, x, y);                            \
    }                                                                                                            \
    void batched_##tag(const Tensor& W, const Tensor* b, const Tensor& X, Tensor& Y) {                           \
        batched_impl(FMT, DT, DNAME, BLOCK, "linear_forward_batched_" #tag "_fp16", W, b, X, Y);                 \
    }
B200_FMT_OPS(q4k, B200Q_FMT_Q4_K, Dtype::Q4_K, "Q4_K", 256)
B200_FMT_OPS(q6k, B200Q_FMT_Q6_K, Dtype::Q6_K, "Q6_K", 256)
B200_FMT_OPS(q8_0, B200Q_FMT_Q8_0, Dtype::Q8_0, "Q8_0", 32)
B200_FMT_OPS(q4_0, B200Q_FMT_Q4_0, Dtype::Q4_0, "Q4_0", 32)
B200_FMT_OPS(q5k, B200Q_FMT_Q5_K, Dtype::Q5_K, "Q5_K", 256)

void embedding_impl(const Tensor& table, const std::int32_t* d_idx, int B, Tensor& out) {
    const char* op = "embedding_lookup_forward";
    int fmt = 0;
    switch (table.dtype) {
        case Dtype::Q4_K: fmt = B200Q_FMT_Q4_K; break;
        case Dtype::Q6_K: fmt = B200Q_FMT_Q6_K; break;
        case Dtype::Q8_0: fmt = B200Q_FMT_Q8_0; break;
        case Dtype::Q4_0: fmt = B200Q_FMT_Q4_0; break;
        case Dtype::Q5_K: fmt = B200Q_FMT_Q5_K; break;
        default: op_fail(op, "table dtype must be Q4_K, Q6_K, Q8_0, Q4_0 or Q5_K (this op is the quantized-table form)");
    }
    if (table.rows <= 0 || table.cols <= 0) op_fail(op, "table has non-positive shape");
    if (B < 0) op_fail(op, "negative batch");
    if (B > 0 && !d_idx) op_fail(op, "null index pointer");
    const bool keep = out.rows == B && out.cols == table.cols && act_dtype(out.dtype) && out.data;
    if (!keep) out.resize(B, table.cols, Dtype::FP16);
    if (B == 0) return;
    check_status(b200q_embedding_gather(layout_fmt(fmt, table), table.data, d_idx, B, table.rows, table.cols, out.data,
                                        static_cast<int>(out.dtype), cuda_current_stream(table.device.index)), op);
}

}  // namespace

// The registration point: what brotensor does in fill_cuda_vtable_specialised
// (src/cuda/concat.cu:359-372) for the same nine slots.
void fill_cuda_tables(OpsVTable& ops, AllocVTable& alloc) {
    ops.linear_forward_group_fp16 = group_impl;
    ops.linear_forward_swiglu_fp16 = swiglu_impl;
    ops.linear_forward_group_rmsnorm_fp16 = group_rmsnorm_impl;
    ops.dequant_q4k_to_fp16 = dequant_q4k;
    ops.linear_forward_q4k_fp16 = gemv_q4k;
    ops.linear_forward_batched_q4k_fp16 = batched_q4k;
    ops.dequant_q8_0_to_fp16 = dequant_q8_0;
    ops.linear_forward_q8_0_fp16 = gemv_q8_0;
    ops.linear_forward_batched_q8_0_fp16 = batched_q8_0;
    ops.dequant_q4_0_to_fp16 = dequant_q4_0;
    ops.linear_forward_q4_0_fp16 = gemv_q4_0;
    ops.linear_forward_batched_q4_0_fp16 = batched_q4_0;
    ops.dequant_q5k_to_fp16 = dequant_q5k;
    ops.linear_forward_q5k_fp16 = gemv_q5k;
    ops.linear_forward_batched_q5k_fp16 = batched_q5k;
    ops.embedding_lookup_forward = embedding_impl;
    ops.dequant_q6k_to_fp16 = dequant_q6k;
    ops.linear_forward_q6k_fp16 = gemv_q6k;
    ops.linear_forward_batched_q6k_fp16 = batched_q6k;
    alloc.alloc = c_alloc; alloc.free = c_free;
    alloc.memcpy_h2d = c_h2d; alloc.memcpy_d2h = c_d2h; alloc.memcpy_h2d_async = c_h2d_async; alloc.memcpy_d2h_async = c_d2h_async; alloc.memcpy_d2d = c_d2d; alloc.memcpy_peer = c_peer;
    alloc.memset_zero = c_zero; alloc.sync = c_sync; alloc.mem_info = c_mem_info; alloc.device_name = c_name;
}

}  // namespace brotensor_b200::detail

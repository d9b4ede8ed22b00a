// C-ABI entry points (include/b200q.h): argument validation, routing between
// kernels and error reporting. No compute happens on the host and nothing here
// falls back to a CPU path.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace b200q {

int launch_dequant(int fmt, const void* W, void* out, int out_dtype, int64_t rows, int K, cudaStream_t st);
int launch_gather(int fmt, const void* W, const int32_t* idx, void* out, int out_dtype, int B, int64_t rows, int K, cudaStream_t st);
int launch_repack(int fmt, const void* src, void* dst, int64_t rows, int K, bool to_runs, cudaStream_t st);
int launch_gemv_simple(int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype,
                       int M, int N, int K, cudaStream_t st);
int launch_gemv_stream(int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype,
                       int M, int N, int K, int sms, size_t smem_max, int* status, cudaStream_t st, bool* taken);
int launch_gemv_dp(int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype, int M,
                   int N, int K, int sms, size_t smem_max, int* status, cudaStream_t st, bool* taken, const ShardOut* sh);
int launch_gemv_dp_multi(int fmt, int n_seg, const void* const* W, const int* N, void* const* Y, const void* const* bias,
                         const void* X, int x_dtype, int y_dtype, int K, int sms, size_t smem_max, int* status, cudaStream_t st,
                         bool* taken, const void* gamma, float eps);
int launch_gemv_dp_swiglu(int fmt, const void* Wg, const void* Wu, const void* X, int x_dtype, void* Y, int y_dtype, int N, int K,
                          int sms, size_t smem_max, int* status, cudaStream_t st, bool* taken);
void stream_set_option(int which, int value);
void gemm_set_pair(int v);
int gemm_get_pair();
void gemm_set_split(int v);
int gemm_get_split();
void dp_set_groups(int v);
void dp_set_tile_pairs(int v);
void dp_set_split_full(int v);
void dp_set_wait_limit_us(int v);
void dp_set_lean(int v);
void dp_set_step_fill(int v);
int launch_gemv_xr(int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype, int M, int N, int K,
                   int sms, int* status, cudaStream_t st, bool* taken);
int launch_gemv_i8(int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype, int M, int N, int K,
                   int sms, int* status, cudaStream_t st, bool* taken);
void i8_set_enabled(int v);
int i8_get_enabled();
void xr_set_enabled(int v);
int xr_get_enabled();
int dp_get_wait_limit_us();
int dp_get_tile_pairs();
int dp_get_groups();
int stream_get_option(int which);
size_t gemm_tc_workspace_bytes(int fmt, int x_dtype, int M, int N, int K);
int launch_gemm_tc(int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype, int M,
                   int N, int K, void* ws, size_t ws_bytes, int sms, int* status, cudaStream_t st, bool* taken);

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

// One status word per device, living in the module's global memory.
__device__ int g_dev_status;

constexpr int kMaxDev = 64;
struct DevInfo {
    std::atomic<bool> ready{false};  // set last, with release ordering: a thread that sees it sees the fields below
    int sms = 0;
    size_t smem_optin = 0;
    int* status = nullptr;
    std::atomic<unsigned long long> tc_calls[3];
};
static DevInfo g_dev[kMaxDev];
static std::mutex g_dev_mu;

static int fmt_slot(int fmt) { return fmt == kQ4_K ? 0 : (fmt == kQ6_K || fmt == kQ6_KP) ? 1 : fmt == kQ8_0 ? 2 : -1; }

static int dev_info(DevInfo** out) {
    int dev = -1;
    B200Q_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDev) return fail(B200Q_ERR_CUDA, "device ordinal %d out of range", dev);
    DevInfo& d = g_dev[dev];
    if (!d.ready.load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lk(g_dev_mu);
        if (!d.ready.load(std::memory_order_relaxed)) {
            int sms = 0, smem = 0;
            B200Q_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
            B200Q_CUDA_TRY(cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
            void* p = nullptr;
            B200Q_CUDA_TRY(cudaGetSymbolAddress(&p, g_dev_status));
            d.sms = sms;
            d.smem_optin = (size_t)smem;
            d.status = static_cast<int*>(p);
            for (auto& c : d.tc_calls) c.store(0);
            d.ready.store(true, std::memory_order_release);
        }
    }
    *out = &d;
    return B200Q_OK;
}

int* device_status_word(int dev) { return (dev >= 0 && dev < kMaxDev && g_dev[dev].ready.load(std::memory_order_acquire)) ? g_dev[dev].status : nullptr; }

static int g_opt_gemv_path = 0;
static int g_opt_gemm_path = 0;

static bool dt_ok(int dt) { return dt == B200Q_DT_F32 || dt == B200Q_DT_F16 || dt == B200Q_DT_BF16; }
static int dt_size(int dt) { return dt == B200Q_DT_F32 ? 4 : 2; }
static bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
// Alignment a weight pointer needs for its block header loads.
static size_t w_align(int fmt) { return fmt == kQ6_KP ? 16 : (fmt == kQ4_K || fmt == kQ5_K) ? 4 : 2; }
// Formats the streaming decode kernels, the tensor-core GEMM and the fused / sharded forms take; the
// others (Q4_0, Q5_K) run through the plain-load GEMV.
static bool streaming_fmt(int fmt) { return fmt == kQ4_K || fmt == kQ6_K || fmt == kQ6_KP || fmt == kQ8_0; }

static int check_linear_args(const char* op, int fmt, const void* W, const void* X, int x_dtype, const void* Y,
                             int y_dtype, int M, int N, int K) {
    const int be = b200q_block_elems(fmt);
    if (!be) return fail(B200Q_ERR_BAD_ARG, "%s: unknown block format %d", op, fmt);
    if (!dt_ok(x_dtype) || !dt_ok(y_dtype)) return fail(B200Q_ERR_BAD_ARG, "%s: unknown dtype (x %d, y %d)", op, x_dtype, y_dtype);
    if (M < 0 || N < 0 || K <= 0) return fail(B200Q_ERR_BAD_ARG, "%s: negative shape (M %d, N %d, K %d)", op, M, N, K);
    if (K % be) return fail(B200Q_ERR_BAD_ARG, "%s: K (%d) must be a multiple of %d", op, K, be);
    if (fmt == kQ6_KP && K % kQ6RunElems) return fail(B200Q_ERR_BAD_ARG, "%s: K (%d) must be a multiple of %d for repacked Q6_K", op, K, kQ6RunElems);
    if (M == 0 || N == 0) return B200Q_OK;
    if (!W || !X || !Y) return fail(B200Q_ERR_BAD_ARG, "%s: null pointer", op);
    if (!aligned(W, w_align(fmt))) return fail(B200Q_ERR_BAD_ARG, "%s: W is not aligned to its block header", op);
    if (!aligned(X, 16)) return fail(B200Q_ERR_BAD_ARG, "%s: X must be 16-byte aligned", op);
    if (!aligned(Y, (size_t)dt_size(y_dtype))) return fail(B200Q_ERR_BAD_ARG, "%s: Y is not aligned to its element size", op);
    return B200Q_OK;
}

}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_abi_version(void) { return 1; }

const char* b200q_status_str(int s) {
    switch (s) {
        case B200Q_OK: return "ok";
        case B200Q_ERR_BAD_ARG: return "bad argument";
        case B200Q_ERR_UNSUPPORTED: return "unsupported shape or layout";
        case B200Q_ERR_CUDA: return "CUDA error";
        case B200Q_ERR_TIMEOUT: return "device-side wait timed out";
        case B200Q_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    }
    return "unknown status";
}

const char* b200q_last_error(void) { return g_err; }

int b200q_block_elems(int fmt) {
    return (fmt == kQ8_0 || fmt == kQ4_0) ? 32 : (fmt == kQ4_K || fmt == kQ6_K || fmt == kQ6_KP || fmt == kQ5_K) ? 256 : 0;
}
int b200q_block_bytes(int fmt) {
    return fmt == kQ8_0 ? 34 : fmt == kQ4_0 ? 18 : fmt == kQ4_K ? 144 : fmt == kQ5_K ? 176 : (fmt == kQ6_K || fmt == kQ6_KP) ? 210 : 0;
}
size_t b200q_packed_bytes(int fmt, int64_t rows, int K) {
    const int be = b200q_block_elems(fmt);
    if (!be || rows < 0 || K < 0 || K % be) return 0;
    return (size_t)rows * (size_t)(K / be) * (size_t)b200q_block_bytes(fmt);
}

int b200q_repacked_fmt(int fmt, int K) { return (fmt == kQ6_K && K > 0 && K % kQ6RunElems == 0) ? kQ6_KP : fmt; }

static int repack_common(const char* op, int fmt, const void* src, void* dst, int64_t rows, int K, bool to_runs, void* stream) {
    const int be = (fmt == kQ6_KP) ? 0 : b200q_block_elems(fmt);
    if (!be) return fail(B200Q_ERR_BAD_ARG, "%s: fmt (%d) must be a raw block format", op, fmt);
    if (rows < 0 || K <= 0 || K % be) return fail(B200Q_ERR_BAD_ARG, "%s: K (%d) must be a positive multiple of %d", op, K, be);
    if (rows == 0) return B200Q_OK;
    if (!src || !dst) return fail(B200Q_ERR_BAD_ARG, "%s: null pointer", op);
    DevInfo* d;
    if (int rc = dev_info(&d)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (b200q_repacked_fmt(fmt, K) != fmt) {
        if (!aligned(src, 2) || !aligned(dst, 2)) return fail(B200Q_ERR_BAD_ARG, "%s: pointers must be 2-byte aligned", op);
        return launch_repack(fmt, src, dst, rows, K, to_runs, st);
    }
    if (src != dst) B200Q_CUDA_TRY(cudaMemcpyAsync(dst, src, b200q_packed_bytes(fmt, rows, K), cudaMemcpyDeviceToDevice, st));
    return B200Q_OK;
}
int b200q_repack(int fmt, const void* src, void* dst, int64_t rows, int K, void* stream) {
    return repack_common("repack", fmt, src, dst, rows, K, true, stream);
}
int b200q_unpack(int fmt, const void* src, void* dst, int64_t rows, int K, void* stream) {
    return repack_common("unpack", fmt, src, dst, rows, K, false, stream);
}

int b200q_dequant(int fmt, const void* W, void* out, int out_dtype, int64_t rows, int K, void* stream) {
    const int be = b200q_block_elems(fmt);
    if (!be) return fail(B200Q_ERR_BAD_ARG, "dequant: unknown block format %d", fmt);
    if (!dt_ok(out_dtype)) return fail(B200Q_ERR_BAD_ARG, "dequant: unknown output dtype %d", out_dtype);
    if (rows < 0 || K <= 0 || K % be) return fail(B200Q_ERR_BAD_ARG, "dequant: K (%d) must be a positive multiple of %d", K, be);
    if (fmt == kQ6_KP && K % kQ6RunElems) return fail(B200Q_ERR_BAD_ARG, "dequant: K (%d) must be a multiple of %d for repacked Q6_K", K, kQ6RunElems);
    if (rows == 0) return B200Q_OK;
    if (!W || !out) return fail(B200Q_ERR_BAD_ARG, "dequant: null pointer");
    if (!aligned(W, w_align(fmt))) return fail(B200Q_ERR_BAD_ARG, "dequant: W is not aligned to its block header");
    if (!aligned(out, 16)) return fail(B200Q_ERR_BAD_ARG, "dequant: output must be 16-byte aligned");
    DevInfo* d;
    if (int rc = dev_info(&d)) return rc;
    return launch_dequant(fmt, W, out, out_dtype, rows, K, static_cast<cudaStream_t>(stream));
}

int b200q_embedding_gather(int fmt, const void* table, const int32_t* idx, int B, int64_t rows, int K, void* out, int out_dtype,
                           void* stream) {
    const int be = b200q_block_elems(fmt);
    if (!be) return fail(B200Q_ERR_BAD_ARG, "embedding_gather: unknown block format %d", fmt);
    if (!dt_ok(out_dtype)) return fail(B200Q_ERR_BAD_ARG, "embedding_gather: unknown output dtype %d", out_dtype);
    if (B < 0 || rows < 0 || K <= 0 || K % be || K % 8) return fail(B200Q_ERR_BAD_ARG, "embedding_gather: K (%d) must be a positive multiple of %d", K, be > 8 ? be : 8);
    if (fmt == kQ6_KP && K % kQ6RunElems) return fail(B200Q_ERR_BAD_ARG, "embedding_gather: K (%d) must be a multiple of %d for repacked Q6_K", K, kQ6RunElems);
    if (B == 0) return B200Q_OK;
    if (!table || !idx || !out) return fail(B200Q_ERR_BAD_ARG, "embedding_gather: null pointer");
    if (!aligned(table, w_align(fmt))) return fail(B200Q_ERR_BAD_ARG, "embedding_gather: table is not aligned to its block header");
    if (!aligned(idx, 4)) return fail(B200Q_ERR_BAD_ARG, "embedding_gather: idx must be 4-byte aligned");
    if (!aligned(out, 16)) return fail(B200Q_ERR_BAD_ARG, "embedding_gather: output must be 16-byte aligned");
    DevInfo* d;
    if (int rc = dev_info(&d)) return rc;
    return launch_gather(fmt, table, idx, out, out_dtype, B, rows, K, static_cast<cudaStream_t>(stream));
}

// The streaming kernel for a decode GEMV of M <= 8 rows, by measurement on B200 (14336 x 4096 and
// 4096 x 14336, us per launch): the integer-dot kernel's work grows with M, the warp-MMA kernel's
// hardly does - Q4_K 8.1 / 12.8 / 16.1 / 21.9 at one to four rows against 16.7 / 18.3 / 19.9 / 21.3
// with warp MMA, Q8_0 11.7 / 16.3 / 19.4 / 23.5 against 18.6 / 18.7 / 19.0 / 19.8 - so warp MMA takes
// over at four rows (Q8_0: three) and is the only one for five to eight.
// *taken = false when neither kernel takes the shape.
static int gemv_streaming(DevInfo* d, int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y,
                          int y_dtype, int M, int N, int K, cudaStream_t st, bool* taken) {
    *taken = false;
    const size_t smem = d->smem_optin - 1024;
    if (M >= 2) {  // Q8_0, K = 2048 / 4096: the integer tensor-core kernel streams at the one-row rate for any M <= 8
        if (int rc = launch_gemv_i8(fmt, W, X, x_dtype, bias, Y, y_dtype, M, N, K, d->sms, d->status, st, taken)) return rc;
        if (*taken) return B200Q_OK;
    }
    const bool mma_first = M >= (fmt == kQ8_0 ? 3 : 4);
    if (mma_first) {
        if (int rc = launch_gemv_stream(fmt, W, X, x_dtype, bias, Y, y_dtype, M, N, K, d->sms, smem, d->status, st, taken)) return rc;
        if (*taken) return B200Q_OK;
    }
    if (M == 1) {
        if (int rc = launch_gemv_xr(fmt, W, X, x_dtype, bias, Y, y_dtype, M, N, K, d->sms, d->status, st, taken)) return rc;
        if (*taken) return B200Q_OK;
    }
    if (M <= 4) {
        if (int rc = launch_gemv_dp(fmt, W, X, x_dtype, bias, Y, y_dtype, M, N, K, d->sms, smem, d->status, st, taken, nullptr)) return rc;
        if (*taken) return B200Q_OK;
    }
    if (!mma_first) {
        if (int rc = launch_gemv_stream(fmt, W, X, x_dtype, bias, Y, y_dtype, M, N, K, d->sms, smem, d->status, st, taken)) return rc;
    }
    return B200Q_OK;
}

int b200q_gemv(int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype, int M,
               int N, int K, void* stream) {
    if (int rc = check_linear_args("gemv", fmt, W, X, x_dtype, Y, y_dtype, M, N, K)) return rc;
    if (M > 8) return fail(B200Q_ERR_UNSUPPORTED, "gemv: M (%d) exceeds 8 activation rows; use b200q_gemm", M);
    if (M == 0 || N == 0) return B200Q_OK;
    DevInfo* d;
    if (int rc = dev_info(&d)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!streaming_fmt(fmt)) return launch_gemv_simple(fmt, W, X, x_dtype, bias, Y, y_dtype, M, N, K, st);
    // 0 = automatic, 1 = plain-load kernel, 2 = warp-MMA streaming kernel, 3 = integer-dot streaming kernel
    if (g_opt_gemv_path == 0) {
        bool taken = false;
        if (int rc = gemv_streaming(d, fmt, W, X, x_dtype, bias, Y, y_dtype, M, N, K, st, &taken)) return rc;
        if (taken) return B200Q_OK;
        if (M > 4) {
            // Eight activation rows of a long K do not fit beside the weight ring (K = 14336): two
            // passes of up to four rows through the streaming kernels still read the weights at
            // the stream rate, which the plain-load kernel does not.
            if (int rc = gemv_streaming(d, fmt, W, X, x_dtype, bias, Y, y_dtype, 4, N, K, st, &taken)) return rc;
            if (taken) {
                const size_t xs = (size_t)K * dt_size(x_dtype), ys = (size_t)N * dt_size(y_dtype);
                const void* X2 = static_cast<const uint8_t*>(X) + 4 * xs;
                void* Y2 = static_cast<uint8_t*>(Y) + 4 * ys;
                if (int rc = gemv_streaming(d, fmt, W, X2, x_dtype, bias, Y2, y_dtype, M - 4, N, K, st, &taken)) return rc;
                if (taken) return B200Q_OK;
                return launch_gemv_simple(fmt, W, X2, x_dtype, bias, Y2, y_dtype, M - 4, N, K, st);
            }
        }
    }
    if (g_opt_gemv_path == 3) {
        bool taken = false;
        if (int rc = launch_gemv_dp(fmt, W, X, x_dtype, bias, Y, y_dtype, M, N, K, d->sms, d->smem_optin - 1024, d->status, st, &taken, nullptr))
            return rc;
        if (taken) return B200Q_OK;
        return fail(B200Q_ERR_UNSUPPORTED, "gemv: shape (M %d, N %d, K %d, fmt %d) is outside the integer-dot kernel", M, N, K, fmt);
    }
    if (g_opt_gemv_path == 2) {
        bool taken = false;
        if (int rc = launch_gemv_stream(fmt, W, X, x_dtype, bias, Y, y_dtype, M, N, K, d->sms, d->smem_optin - 1024, d->status, st, &taken))
            return rc;
        if (taken) return B200Q_OK;
        return fail(B200Q_ERR_UNSUPPORTED, "gemv: shape (M %d, N %d, K %d, fmt %d) is outside the streaming kernel", M, N, K, fmt);
    }
    return launch_gemv_simple(fmt, W, X, x_dtype, bias, Y, y_dtype, M, N, K, st);
}

int b200q_gemv_swiglu(int fmt, const void* W_gate, const void* W_up, const void* x, int x_dtype, void* y, int y_dtype,
                      int N, int K, void* stream) {
    if (b200q_block_elems(fmt) && !streaming_fmt(fmt)) return fail(B200Q_ERR_UNSUPPORTED, "gemv_swiglu: block format %d has no fused form", fmt);
    if (int rc = check_linear_args("gemv_swiglu", fmt, W_gate, x, x_dtype, y, y_dtype, 1, N, K)) return rc;
    if (int rc = check_linear_args("gemv_swiglu", fmt, W_up, x, x_dtype, y, y_dtype, 1, N, K)) return rc;
    if (N == 0) return B200Q_OK;
    DevInfo* d;
    if (int rc = dev_info(&d)) return rc;
    bool taken = false;
    if (int rc = launch_gemv_dp_swiglu(fmt, W_gate, W_up, x, x_dtype, y, y_dtype, N, K, d->sms, d->smem_optin - 1024, d->status,
                                       static_cast<cudaStream_t>(stream), &taken))
        return rc;
    if (!taken)
        return fail(B200Q_ERR_UNSUPPORTED, "gemv_swiglu: shape (N %d, K %d, fmt %d) or weight alignment is outside the streaming kernel", N, K, fmt);
    return B200Q_OK;
}

int b200q_gemv_multi(int fmt, int n, const void* const* W, const int* N, void* const* Y, const void* const* bias,
                     const void* x, int x_dtype, int y_dtype, int K, void* stream) {
    if (n < 1 || n > kMaxSegments) return fail(B200Q_ERR_BAD_ARG, "gemv_multi: %d matrices (1..%d)", n, kMaxSegments);
    if (!W || !N || !Y) return fail(B200Q_ERR_BAD_ARG, "gemv_multi: null table");
    for (int s = 0; s < n; ++s) {
        if (N[s] <= 0) return fail(B200Q_ERR_BAD_ARG, "gemv_multi: matrix %d has %d rows", s, N[s]);
        if (int rc = check_linear_args("gemv_multi", fmt, W[s], x, x_dtype, Y[s], y_dtype, 1, N[s], K)) return rc;
    }
    DevInfo* d;
    if (int rc = dev_info(&d)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (n > 1 && streaming_fmt(fmt) && (g_opt_gemv_path == 0 || g_opt_gemv_path == 3)) {
        bool taken = false;
        if (int rc = launch_gemv_dp_multi(fmt, n, W, N, Y, bias, x, x_dtype, y_dtype, K, d->sms, d->smem_optin - 1024, d->status, st, &taken, nullptr, 0.f))
            return rc;
        if (taken) return B200Q_OK;
    }
    // shapes the grouped kernel does not take: one launch per matrix
    for (int s = 0; s < n; ++s)
        if (int rc = b200q_gemv(fmt, W[s], x, x_dtype, bias ? bias[s] : nullptr, Y[s], y_dtype, 1, N[s], K, stream)) return rc;
    return B200Q_OK;
}

int b200q_gemv_multi_rmsnorm(int fmt, int n, const void* const* W, const int* N, void* const* Y, const void* const* bias,
                             const void* x, int x_dtype, const void* gamma, float eps, int y_dtype, int K, void* stream) {
    if (n < 1 || n > kMaxSegments) return fail(B200Q_ERR_BAD_ARG, "gemv_multi_rmsnorm: %d matrices (1..%d)", n, kMaxSegments);
    if (!W || !N || !Y) return fail(B200Q_ERR_BAD_ARG, "gemv_multi_rmsnorm: null table");
    if (b200q_block_elems(fmt) && !streaming_fmt(fmt)) return fail(B200Q_ERR_UNSUPPORTED, "gemv_multi_rmsnorm: block format %d has no fused form", fmt);
    if (!gamma || !aligned(gamma, 16)) return fail(B200Q_ERR_BAD_ARG, "gemv_multi_rmsnorm: gamma must be a 16-byte aligned vector of K elements");
    if (!(eps >= 0.f)) return fail(B200Q_ERR_BAD_ARG, "gemv_multi_rmsnorm: eps must not be negative");
    for (int s = 0; s < n; ++s) {
        if (N[s] <= 0) return fail(B200Q_ERR_BAD_ARG, "gemv_multi_rmsnorm: matrix %d has %d rows", s, N[s]);
        if (int rc = check_linear_args("gemv_multi_rmsnorm", fmt, W[s], x, x_dtype, Y[s], y_dtype, 1, N[s], K)) return rc;
    }
    DevInfo* d;
    if (int rc = dev_info(&d)) return rc;
    bool taken = false;
    if (int rc = launch_gemv_dp_multi(fmt, n, W, N, Y, bias, x, x_dtype, y_dtype, K, d->sms, d->smem_optin - 1024, d->status,
                                      static_cast<cudaStream_t>(stream), &taken, gamma, eps))
        return rc;
    if (!taken)
        return fail(B200Q_ERR_UNSUPPORTED, "gemv_multi_rmsnorm: shape (K %d, fmt %d) or weight alignment is outside the streaming kernel", K, fmt);
    return B200Q_OK;
}

static int gemv_shard_impl(const char* name, int fmt, const void* W_shard, const void* x, int x_dtype, const void* bias_shard, int rows,
                           int K, int row_offset, int total_rows, int rank, int world, void* const* peer_out,
                           void* const* peer_cand, void* state, int k, void* top_val, void* top_idx, void* stream) {
    if (b200q_block_elems(fmt) && !streaming_fmt(fmt)) return fail(B200Q_ERR_UNSUPPORTED, "%s: block format %d has no sharded form", name, fmt);
    static float dummy_y;  // check_linear_args wants a non-null result pointer; the sharded form has none
    if (int rc = check_linear_args(name, fmt, W_shard, x, x_dtype, &dummy_y, B200Q_DT_F32, 1, rows, K)) return rc;
    if (world < 1 || world > kMaxShardRanks || rank < 0 || rank >= world)
        return fail(B200Q_ERR_BAD_ARG, "%s: rank %d of %d (at most %d ranks)", name, rank, world, kMaxShardRanks);
    if (row_offset < 0 || total_rows <= 0 || (long long)row_offset + rows > total_rows)
        return fail(B200Q_ERR_BAD_ARG, "%s: rows [%d, %d) do not lie in [0, %d)", name, row_offset, row_offset + rows, total_rows);
    if (!peer_out || !state) return fail(B200Q_ERR_BAD_ARG, "%s: null peer table or state", name);
    for (int q = 0; q < world; ++q)
        if (!peer_out[q]) return fail(B200Q_ERR_BAD_ARG, "%s: null pointer for rank %d", name, q);
    if (rows == 0) return fail(B200Q_ERR_UNSUPPORTED, "%s: an empty shard cannot signal its arrival", name);
    if (k) {
        if (k < 1 || k > kMaxTopK) return fail(B200Q_ERR_BAD_ARG, "%s: k = %d candidates (1 .. %d)", name, k, kMaxTopK);
        if (!peer_cand || !top_val || !top_idx) return fail(B200Q_ERR_BAD_ARG, "%s: null candidate table or result", name);
        if (total_rows >= 0xFFFFF) return fail(B200Q_ERR_UNSUPPORTED, "%s: a candidate's row has 20 bits (%d rows)", name, total_rows);
        for (int q = 0; q < world; ++q)
            if (!peer_cand[q]) return fail(B200Q_ERR_BAD_ARG, "%s: null candidate table for rank %d", name, q);
    }
    DevInfo* d;
    if (int rc = dev_info(&d)) return rc;
    ShardOut sh;
    sh.world = world;
    sh.rank = rank;
    sh.row_offset = row_offset;
    sh.total_rows = total_rows;
    sh.out = reinterpret_cast<float* const*>(peer_out);
    sh.state = static_cast<unsigned int*>(state);
    sh.topk = k;
    sh.cand = reinterpret_cast<uint32_t* const*>(peer_cand);
    sh.top_val = static_cast<float*>(top_val);
    sh.top_idx = static_cast<int*>(top_idx);
    bool taken = false;
    if (int rc = launch_gemv_dp(fmt, W_shard, x, x_dtype, bias_shard, nullptr, B200Q_DT_F32, 1, rows, K, d->sms,
                                d->smem_optin - 1024, d->status, static_cast<cudaStream_t>(stream), &taken, &sh))
        return rc;
    if (!taken)
        return fail(B200Q_ERR_UNSUPPORTED, "%s: shape (rows %d, K %d, fmt %d) or weight alignment is outside the streaming kernel", name, rows, K, fmt);
    return B200Q_OK;
}

int b200q_gemv_shard(int fmt, const void* W_shard, const void* x, int x_dtype, const void* bias_shard, int rows, int K,
                     int row_offset, int total_rows, int rank, int world, void* const* peer_out, void* state, void* stream) {
    return gemv_shard_impl("gemv_shard", fmt, W_shard, x, x_dtype, bias_shard, rows, K, row_offset, total_rows, rank, world, peer_out,
                           nullptr, state, 0, nullptr, nullptr, stream);
}

int b200q_gemv_shard_topk(int fmt, const void* W_shard, const void* x, int x_dtype, const void* bias_shard, int rows, int K,
                          int row_offset, int total_rows, int rank, int world, void* const* peer_out,
                          void* const* peer_cand, void* state, int k, void* top_val, void* top_idx, void* stream) {
    if (k < 1) return fail(B200Q_ERR_BAD_ARG, "gemv_shard_topk: k = %d candidates (1 .. %d)", k, kMaxTopK);
    return gemv_shard_impl("gemv_shard_topk", fmt, W_shard, x, x_dtype, bias_shard, rows, K, row_offset, total_rows, rank, world,
                           peer_out, peer_cand, state, k, top_val, top_idx, stream);
}

size_t b200q_gemm_workspace_bytes(int fmt, int x_dtype, int M, int N, int K) {
    if (!b200q_block_elems(fmt) || M <= 0 || N <= 0 || K <= 0) return 0;
    return gemm_tc_workspace_bytes(fmt, x_dtype, M, N, K);
}

int b200q_gemm(int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype, int M,
               int N, int K, void* ws, size_t ws_bytes, void* stream) {
    if (int rc = check_linear_args("gemm", fmt, W, X, x_dtype, Y, y_dtype, M, N, K)) return rc;
    if (M == 0 || N == 0) return B200Q_OK;
    DevInfo* d;
    if (int rc = dev_info(&d)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // Nine to sixteen rows: the tensor-core GEMM's producers decode the whole matrix for however few tokens
    // (14336 x 4096: 46-48 us for any M up to 32), two passes of the small-batch GEMV on the integer tensor
    // cores take 28-30 us (Q4_K, Q8_0; 4096 x 4096: 14-15 against 18-20), and for Q6_K from 8192 rows two
    // passes of the warp-MMA GEMV 53-55 against 67. From 24 rows the GEMM is the faster one.
    if (g_opt_gemm_path == 0 && M > 8 && M <= 16 && K <= 4096 &&
        (((fmt == kQ4_K || fmt == kQ8_0) && (K == 2048 || K == 4096) && i8_get_enabled()) || (fmt == kQ6_K && N >= 8192))) {
        const size_t xs = (size_t)dt_size(x_dtype) * K, ys = (size_t)dt_size(y_dtype) * N;
        for (int m0 = 0; m0 < M; m0 += 8) {
            const int mm = M - m0 < 8 ? M - m0 : 8;
            if (int rc = b200q_gemv(fmt, W, static_cast<const char*>(X) + xs * m0, x_dtype, bias,
                                    static_cast<char*>(Y) + ys * m0, y_dtype, mm, N, K, stream))
                return rc;
        }
        d->tc_calls[fmt_slot(fmt)].fetch_add(1);  // mma.sync on the tensor cores, int8 or FP16
        return B200Q_OK;
    }
    if (g_opt_gemm_path != 1) {
        bool taken = false;
        if (int rc = launch_gemm_tc(fmt, W, X, x_dtype, bias, Y, y_dtype, M, N, K, ws, ws_bytes, d->sms, d->status, st, &taken))
            return rc;
        if (taken) {
            d->tc_calls[fmt_slot(fmt)].fetch_add(1);
            return B200Q_OK;
        }
        if (g_opt_gemm_path == 2)
            return fail(B200Q_ERR_UNSUPPORTED, "gemm: shape (M %d, N %d, K %d, fmt %d) is outside the tensor-core kernel", M, N, K, fmt);
    }
    // Shapes the tensor-core kernel does not take: passes of up to 8 activation rows
    // through the decode GEMV (W is re-read once per pass).
    const size_t xs = (size_t)dt_size(x_dtype) * K, ys = (size_t)dt_size(y_dtype) * N;
    for (int m0 = 0; m0 < M; m0 += 8) {
        const int mm = M - m0 < 8 ? M - m0 : 8;
        if (int rc = b200q_gemv(fmt, W, static_cast<const char*>(X) + xs * m0, x_dtype, bias,
                                static_cast<char*>(Y) + ys * m0, y_dtype, mm, N, K, stream))
            return rc;
    }
    return B200Q_OK;
}

int b200q_linear(int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype, int M,
                 int N, int K, void* ws, size_t ws_bytes, void* stream) {
    if (M <= 8) return b200q_gemv(fmt, W, X, x_dtype, bias, Y, y_dtype, M, N, K, stream);
    return b200q_gemm(fmt, W, X, x_dtype, bias, Y, y_dtype, M, N, K, ws, ws_bytes, stream);
}

unsigned long long b200q_tc_calls_consume(int fmt) {
    const int s = fmt_slot(fmt);
    int dev = -1;
    if (s < 0 || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return 0;
    return g_dev[dev].tc_calls[s].exchange(0);
}
unsigned long long brotensor_q4k_wmma_calls_consume(void) { return b200q_tc_calls_consume(kQ4_K); }
unsigned long long brotensor_q6k_wmma_calls_consume(void) { return b200q_tc_calls_consume(kQ6_K); }
unsigned long long brotensor_q8_0_wmma_calls_consume(void) { return b200q_tc_calls_consume(kQ8_0); }

int b200q_device_status(int* status_out) {
    DevInfo* d;
    if (int rc = dev_info(&d)) return rc;
    B200Q_CUDA_TRY(cudaDeviceSynchronize());
    int v = 0;
    B200Q_CUDA_TRY(cudaMemcpy(&v, d->status, sizeof(int), cudaMemcpyDeviceToHost));
    if (v != 0) {
        const int zero = 0;
        B200Q_CUDA_TRY(cudaMemcpy(d->status, &zero, sizeof(int), cudaMemcpyHostToDevice));
    }
    if (status_out) *status_out = v;
    if (v != 0) return fail(B200Q_ERR_TIMEOUT, "a kernel's bounded wait ran out (device status %d)", v);
    return B200Q_OK;
}

int b200q_set_option(const char* key, int value) {
    if (!key) return fail(B200Q_ERR_BAD_ARG, "set_option: null key");
    if (!strcmp(key, "gemv_path")) g_opt_gemv_path = value;
    else if (!strcmp(key, "gemm_path")) g_opt_gemm_path = value;
    else if (!strcmp(key, "gemv_stages")) stream_set_option(0, value);
    else if (!strcmp(key, "pdl")) stream_set_option(1, value);
    else if (!strcmp(key, "gemv_stage_kb")) stream_set_option(2, value);
    else if (!strcmp(key, "gemv_grid")) stream_set_option(3, value);
    else if (!strcmp(key, "gemv_groups")) dp_set_groups(value);
    else if (!strcmp(key, "gemv_tile_pairs")) dp_set_tile_pairs(value);
    else if (!strcmp(key, "gemv_split_full")) dp_set_split_full(value);
    else if (!strcmp(key, "gemm_pair")) gemm_set_pair(value);
    else if (!strcmp(key, "gemm_split")) gemm_set_split(value);
    else if (!strcmp(key, "wait_limit_us")) dp_set_wait_limit_us(value);
    else if (!strcmp(key, "gemv_lean")) dp_set_lean(value);
    else if (!strcmp(key, "gemv_xr")) xr_set_enabled(value);
    else if (!strcmp(key, "gemv_i8")) i8_set_enabled(value);
    else if (!strcmp(key, "gemv_step_fill")) dp_set_step_fill(value);
    else return fail(B200Q_ERR_BAD_ARG, "set_option: unknown key '%s'", key);
    return B200Q_OK;
}
int b200q_get_option(const char* key, int* out) {
    if (!key || !out) return fail(B200Q_ERR_BAD_ARG, "get_option: null argument");
    if (!strcmp(key, "gemv_path")) *out = g_opt_gemv_path;
    else if (!strcmp(key, "gemm_path")) *out = g_opt_gemm_path;
    else if (!strcmp(key, "gemv_stages")) *out = stream_get_option(0);
    else if (!strcmp(key, "pdl")) *out = stream_get_option(1);
    else if (!strcmp(key, "gemv_stage_kb")) *out = stream_get_option(2);
    else if (!strcmp(key, "gemv_grid")) *out = stream_get_option(3);
    else if (!strcmp(key, "gemv_groups")) *out = dp_get_groups();
    else if (!strcmp(key, "gemv_xr")) *out = xr_get_enabled();
    else if (!strcmp(key, "gemv_i8")) *out = i8_get_enabled();
    else if (!strcmp(key, "gemv_tile_pairs")) *out = dp_get_tile_pairs();
    else if (!strcmp(key, "gemm_pair")) *out = gemm_get_pair();
    else if (!strcmp(key, "gemm_split")) *out = gemm_get_split();
    else if (!strcmp(key, "wait_limit_us")) *out = dp_get_wait_limit_us();
    else return fail(B200Q_ERR_BAD_ARG, "get_option: unknown key '%s'", key);
    return B200Q_OK;
}

}  // extern "C"

// Prefill GEMM for callers that cannot allocate.
//
// b200q_gemm needs scratch for the activation operand image (the FP16, swizzled copy of X
// the tensor-core kernel streams) and asks its caller to own it. Some callers have no
// allocator to ask: code running inside a stream capture (cudaMalloc is not capturable and
// a stream-ordered allocation would become a graph node with its own lifetime rules), a
// serving loop that promised its host a fixed memory footprint after start-up, or a plugin
// slot whose signature has nowhere to carry a workspace pointer. For those this file keeps
// the scratch in the module's own global memory: a fixed array that exists as soon as the
// library is loaded on a device, so the entry point below makes no allocation of any kind,
// device or host, on any call.
//
// The price is the fixed size. kStaticScratchBytes covers 512 tokens of an 8192-wide layer
// (or 1024 tokens at K = 4096); larger problems are refused with B200Q_ERR_WORKSPACE and
// belong to b200q_gemm with a caller-owned workspace.
#include <mutex>

#include "common.cuh"

namespace b200q {

constexpr size_t kStaticScratchBytes = 8u << 20;  // 8 MiB per device

// One array per device (every device that loads this module gets its own instance).
// Nothing in it has to be zero, or anything else, when a call starts: the activation
// pre-pass writes every byte the GEMM kernel later reads, padding rows included.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxScratchDev = 64;
static void* g_scratch_addr[kMaxScratchDev];  // device address of the array, per device
static std::mutex g_scratch_mu;

// Resolves the array's address on the current device, once per device. The lookup has to
// run with that device current, which is the case here: cudaGetDevice names it.
static int static_scratch(void** out) {
    int dev = -1;
    B200Q_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxScratchDev) return fail(B200Q_ERR_CUDA, "gemm_static: device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        B200Q_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
        if (!p) return fail(B200Q_ERR_CUDA, "gemm_static: the scratch array has no address on device %d", dev);
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return B200Q_OK;
}

size_t gemm_tc_workspace_min_bytes(int fmt, int x_dtype, int M, int N, int K);

}  // namespace b200q

extern "C" {

size_t b200q_gemm_static_max_bytes(void) { return b200q::kStaticScratchBytes; }

int b200q_gemm_static(int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype, int M,
                      int N, int K, void* stream) {
    using namespace b200q;
    // Size check first, so that an oversized request fails the same way with or without a device.
    // (the activation image alone: where b200q_gemm would split K through a larger workspace, it runs
    // unsplit in whatever part of the array the image leaves, or split if the partial sums fit too)
    const size_t need = gemm_tc_workspace_min_bytes(fmt, x_dtype, M, N, K);
    if (need > kStaticScratchBytes)
        return fail(B200Q_ERR_WORKSPACE,
                    "gemm_static: M %d x K %d needs %zu bytes of scratch, the built-in array holds %zu; "
                    "use b200q_gemm with a caller-owned workspace",
                    M, K, need, (size_t)kStaticScratchBytes);
    void* scratch = nullptr;
    if (need > 0)
        if (int rc = static_scratch(&scratch)) return rc;
    // Same kernels, same routing and the same argument checks as the caller-workspace form.
    return b200q_gemm(fmt, W, X, x_dtype, bias, Y, y_dtype, M, N, K, scratch, need ? kStaticScratchBytes : 0, stream);
}

}  // extern "C"

// Prefill GEMM on the 5th-generation tensor cores (placeholder translation unit:
// the tcgen05 kernel is added here; until then no shape is taken and the caller
// uses passes of the decode GEMV).
#include "common.cuh"

namespace b200q {

size_t gemm_tc_workspace_bytes(int, int, int, int, int) { return 0; }

int launch_gemm_tc(int, const void*, const void*, int, const void*, void*, int, int, int, int, void*, size_t, int,
                   int*, cudaStream_t, bool* taken) {
    *taken = false;
    return B200Q_OK;
}

}  // namespace b200q

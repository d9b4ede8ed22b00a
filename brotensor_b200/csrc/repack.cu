// Device-side repack of uploaded GGUF rows (sm_100a) and its inverse.
//
// Q6_K is the one format whose stored layout fights the hardware: 210-byte blocks are only 2-byte
// aligned, so a kernel that wants 16-byte loads has to read from the boundary before a block and
// shift. The repacked form regroups every run of eight blocks (1680 bytes, already a multiple of
// 16) by field - ql[8][128], qh[8][64], scales[8][16], d[8] - which puts every field of every block
// on a 16-byte boundary without changing the size of a row or a single bit of content: it is a
// byte permutation inside the run, and unpack is the inverse permutation. Rows are multiples of a
// run (K % 2048 == 0), so the flat sweep below never straddles rows.
//
// One warp moves one run: it reads the run's 840 16-bit units into shared memory, then writes them
// to their new places. Reading the whole run before writing makes the in-place call (dst == src)
// safe. brotensor keeps the raw layout and reads it with 16-bit loads
// (src/cuda/detail/load_align.cuh:21-25, src/cuda/q6k_internal.cuh:70-100).
#include "common.cuh"

namespace b200q {

constexpr int kRepackWarps = 8;

// Offset inside the regrouped run of the byte that the raw layout keeps at offset `o` (even) of block `b`.
__device__ __forceinline__ int q6_run_offset(int b, int o) {
    if (o < 128) return b * 128 + o;
    if (o < 192) return 1024 + b * 64 + (o - 128);
    if (o < 208) return 1536 + b * 16 + (o - 192);
    return 1664 + 2 * b;
}

template <bool TO_RUNS>
__global__ void __launch_bounds__(kRepackWarps * 32) repack_q6k_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                                       long long n_runs) {
    __shared__ unsigned short buf[kRepackWarps][kQ6RunBytes / 2];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long stride = (long long)gridDim.x * kRepackWarps;
    for (long long run = (long long)blockIdx.x * kRepackWarps + warp; run < n_runs; run += stride) {
        const unsigned short* s = reinterpret_cast<const unsigned short*>(src + (size_t)run * kQ6RunBytes);
        unsigned short* d = reinterpret_cast<unsigned short*>(dst + (size_t)run * kQ6RunBytes);
        for (int i = lane; i < kQ6RunBytes / 2; i += 32) buf[warp][i] = s[i];
        __syncwarp();
        // unit i of the RAW layout: block i / 105, byte offset 2 * (i % 105)
        for (int i = lane; i < kQ6RunBytes / 2; i += 32) {
            const int b = i / 105, o = 2 * (i - b * 105);
            const int j = q6_run_offset(b, o) >> 1;  // its unit in the regrouped layout
            if (TO_RUNS) d[j] = buf[warp][i];
            else d[i] = buf[warp][j];
        }
        __syncwarp();
    }
}

// fmt is the raw format; only Q6_K rows made of whole runs have a regrouped form.
int launch_repack(int fmt, const void* src, void* dst, int64_t rows, int K, bool to_runs, cudaStream_t st) {
    if (fmt == kQ6_K && K % kQ6RunElems == 0) {
        const long long n_runs = (long long)rows * (K / kQ6RunElems);
        if (n_runs == 0) return B200Q_OK;
        long long blocks = (n_runs + kRepackWarps - 1) / kRepackWarps;
        if (blocks > 148LL * 64) blocks = 148LL * 64;
        const uint8_t* s = static_cast<const uint8_t*>(src);
        uint8_t* d = static_cast<uint8_t*>(dst);
        if (to_runs) repack_q6k_kernel<true><<<(unsigned)blocks, kRepackWarps * 32, 0, st>>>(s, d, n_runs);
        else repack_q6k_kernel<false><<<(unsigned)blocks, kRepackWarps * 32, 0, st>>>(s, d, n_runs);
        B200Q_CUDA_TRY(cudaGetLastError());
        return B200Q_OK;
    }
    return fail(B200Q_ERR_UNSUPPORTED, "repack: format %d with K %d has no regrouped form", fmt, K);
}

}  // namespace b200q

// Pieces shared by the two streaming decode-GEMV kernels (gemv_stream.cu: warp-MMA
// consumers for 5..8 activation rows; gemv_dp.cu: integer dot-product consumers for
// 1..4 rows): launch parameters, the shared-memory ring geometry, the bounded
// mbarrier wait and the producer warp that streams weight rows with bulk copies.
#pragma once

#include "common.cuh"

namespace b200q {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kStreamThreads = kConsumerThreads + 32;  // + producer warp
constexpr int kTileRows = 16;
constexpr int kMaxStages = 8;

struct StreamParams {
    const uint8_t* W;
    const void* X;
    const void* bias;
    void* Y;
    int* status;
    int M, N, K;
    int x_dtype, y_dtype;  // B200Q_DT_* of X/bias and of Y
    int row_bytes;       // bytes of one weight row
    int chunks_per_row;  // K / chunk elements
    int slice_chunks;    // chunks per stage
    int n_slices;        // stages per row tile
    int row_stride;      // bytes between rows inside a stage (padded)
    int n_stages;        // ring depth
    int n_tiles_total;   // > 0: CTAs own whole 16-row tiles (tile-balanced grid); 0: rows split evenly
    int split_full;      // 1: one full barrier per consumer warp and stage; 0: one per stage
    // The launch's units - whole tiles when n_tiles_total > 0, else rows - over the grid: CTA b has
    // split_q + (b < split_r) of them, starting at b * split_q + min(b, split_r) (no division on the device).
    int split_q, split_r;
    unsigned int wait_limit_us;  // bound of the device-side waits in microseconds (0: one second)
    int step_fill;               // 1: only the first stage of a pipeline is requested ahead of the activation loads
#ifdef B200Q_TRACE
    unsigned long long* trace;  // trace builds: sixteen %globaltimer stamps per CTA of this launch
#endif
    // shared-memory offsets (bytes from the 128-byte aligned base)
    int off_xhi, off_xlo, off_sxhi, off_sxlo, off_red, off_stage;
    // Several weight matrices of one format and K that share the activation vector (n_seg > 1):
    // segment s occupies the virtual rows [16 * seg_tile0[s], 16 * seg_tile0[s] + seg_rows[s]) of the
    // launch; W / Y / bias / N above describe segment 0 when n_seg <= 1.
    // Gate/up pair with a SwiGLU epilogue (W_up != nullptr, M = 1): the launch's virtual rows interleave
    // the two matrices - row 2i is gate row i (in W), row 2i + 1 is up row i (in W_up) - so one warp's
    // row pair is exactly what output i = silu(gate_i . x) * (up_i . x) needs; N counts virtual rows.
    const uint8_t* W_up;
    // RMSNorm folded into the activation staging (norm_gamma != nullptr, M = 1): the kernel stages
    // x[j] * gamma[j] * rsqrt(mean_j x[j]^2 + norm_eps) instead of x; gamma has X's dtype and K elements.
    const void* norm_gamma;
    float norm_eps;
    int n_seg;
    int seg_rows[kMaxSegments];
    int seg_tile0[kMaxSegments + 1];
    const uint8_t* seg_W[kMaxSegments];
    void* seg_Y[kMaxSegments];
    const void* seg_bias[kMaxSegments];
    // Row-sharded output (world > 0): instead of Y, every finished row goes to all ranks'
    // result vectors through peer pointers, followed by an arrival flag per rank.
    int sh_world, sh_rank;       // sh_world == 0: plain GEMV
    int sh_row_offset, sh_total; // first global row of this shard; rows of the whole matrix
    float* sh_out[kMaxShardRanks];         // rank q's result buffers: two vectors of sh_total floats, used alternately, then [2][sh_total] 8-byte transfer words
    unsigned int* sh_state;      // this rank: [0] CTAs finished in this launch, [1] completed launches (epoch)
    // Candidate form of the sharded head (sh_topk = k > 0): rank q's candidate table
    // [2 parities][kMaxShardRanks writers][kShardSlots CTAs][kMaxTopK] 8-byte words and this rank's k results.
    int sh_topk;
    uint32_t* sh_cand[kMaxShardRanks];
    float* sh_top_val;
    int* sh_top_idx;
};

template <int FMT>
struct Chunk {
    static constexpr int blocks = Blk<FMT>::chunk_blocks;
    static constexpr int bytes = Blk<FMT>::bytes * blocks;
    static constexpr int elems = Blk<FMT>::elems * blocks;
    // work units (16 rows x 256 elements) per chunk
    static constexpr int units = elems / 256;
};

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded mbarrier wait with an abort flag shared by the CTA. Returns false when
// the wait was abandoned (by this thread's timeout or because another thread of
// the CTA already gave up). A phase that is complete already costs one try_wait and a branch:
// the timer is read only when the thread has to wait.
// (Measured: the waiting part as a function of its own, not inlined, made every decode GEMV 1 to 10 %
// slower - a kernel with a call in it gets a worse register allocation around its hot loop.)
__device__ __forceinline__ bool wait_or_abort_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                                   uint64_t limit_ns) {
    const uint64_t t0 = global_timer_ns();
    for (;;) {
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (global_timer_ns() - t0 > limit_ns) {
            *abort_flag = 1;
            if (status) atomicCAS(status, 0, code);
            return false;
        }
    }
}
constexpr uint64_t kWaitLimitNs = 1000000000ull;  // one second
template <bool kSpinFirst = false>
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                              int code, uint64_t limit_ns = kWaitLimitNs) {
    // Optional fast path for a single latency-critical thread: non-blocking probes, so a
    // phase that completes soon is seen at once instead of after a parked time slice. Whole
    // warps must not use it: their probes fill the shared-memory pipeline the other warps need.
    if constexpr (kSpinFirst) {
        for (int i = 0; i < 256; ++i)
            if (mbar_test_wait(bar, parity)) return true;
    }
    if (mbar_try_wait(bar, parity)) return true;
    return wait_or_abort_slow(bar, parity, abort_flag, status, code, limit_ns);
}

__device__ __forceinline__ void consumer_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory"); }


// Producer warp: streams the CTA's contiguous row range through the ring, one bulk
// copy per weight row and stage. Weights do not depend on the stream-ordered
// predecessor, so this starts before griddepcontrol.wait.
template <int FMT>
__device__ __forceinline__ void stream_producer(const StreamParams& p, uint32_t smem_base, uint64_t* bar_full,
                                                uint64_t* bar_empty, volatile int* abort_flag, int row_begin,
                                                int row_end, int total_iters, int lane) {
    const int stage_bytes = kTileRows * p.row_stride;
    for (int it = 0; it < total_iters; ++it) {
        const int slot = it % p.n_stages;
        const uint32_t par = ((it / p.n_stages) & 1) ^ 1;
        if (!wait_or_abort(smem_u32(&bar_empty[slot]), par, abort_flag, p.status, kDevTimeoutEmpty)) break;
        const int tile = it / p.n_slices, slice = it - tile * p.n_slices;
        const int row0 = row_begin + tile * kTileRows;
        const int nrows = min(kTileRows, row_end - row0);
        const int c0 = slice * p.slice_chunks;
        const int nch = min(p.slice_chunks, p.chunks_per_row - c0);
        const uint32_t bytes = (uint32_t)nch * Chunk<FMT>::bytes;
        const uint32_t full = smem_u32(&bar_full[slot]);
        if (lane == 0) mbar_arrive_expect_tx(full, bytes * (uint32_t)nrows);
        __syncwarp();
        if (lane < nrows) {
            const uint8_t* src = p.W + (size_t)(row0 + lane) * p.row_bytes + (size_t)c0 * Chunk<FMT>::bytes;
            bulk_g2s(smem_base + p.off_stage + slot * stage_bytes + lane * p.row_stride, src, bytes, full);
        }
    }
}

// Ring geometry for a stage of 16 rows x slice: the largest slice (in chunks) whose
// stage fits `target` bytes, the row stride padded to `pad_mod` (mod 128) so rows
// start in different banks, and as many stages (<= want) as fit `avail`.
template <int FMT>
inline bool plan_ring(StreamParams& p, size_t avail, size_t target, int want_stages, int pad_mod) {
    int sc = p.chunks_per_row;
    if (want_stages < 2) want_stages = 2;
    if (want_stages > kMaxStages) want_stages = kMaxStages;
    for (;;) {
        int rs = sc * Chunk<FMT>::bytes;
        rs += ((pad_mod - (rs % 128)) + 128) % 128;
        const size_t sb = (size_t)kTileRows * rs;
        int ns = (int)(avail / sb);
        if (ns > want_stages) ns = want_stages;
        if ((sb <= target && ns >= 2) || sc == 1) {
            if (ns < 2) return false;
            p.slice_chunks = sc;
            p.row_stride = rs;
            p.n_stages = ns;
            p.n_slices = (p.chunks_per_row + sc - 1) / sc;
            return true;
        }
        sc = (sc + 1) / 2;
    }
}

void stream_set_option(int which, int value);
int stream_get_option(int which);

}  // namespace b200q

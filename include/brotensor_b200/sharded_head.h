// Row-sharded LM head over the GPUs of one node, one process per GPU.
//
// Each rank owns a contiguous row range of a quantized (out, in) matrix and a block of
// "exchange memory": two result vectors of `out` floats, two vectors of 8-byte transfer words and a
// table of sampling candidates.
// The ranks exchange CUDA IPC handles of these blocks once (the caller moves the 64-byte
// handles between processes with whatever it has: torch.distributed, MPI, a file), map each
// other's blocks, and from then on a forward is ONE kernel per rank: the decode GEMV of the
// shard whose epilogue sends every row to all ranks over NVLink as a word that carries the call's
// number, and receives the peers' words the same way (b200q_gemv_shard): no collective library, fence,
// flag or counter on the data path.
// forward_topk is the form for greedy / top-k sampling: k (value, row) candidates per rank cross
// the links instead of the logits (b200q_gemv_shard_topk).
//
// brotensor has no sharded form of this op; it only brings up peer access
// (src/cuda/register.cu:90-103).
#pragma once

#include <array>
#include <cstdint>
#include <vector>

#include "brotensor_b200/tensor.h"

namespace brotensor_b200 {

using IpcHandle = std::array<unsigned char, 64>;

class ShardedHead {
public:
    // W_shard: this rank's rows (row_offset .. row_offset + W_shard.rows) of a matrix with
    // total_rows rows; lives on the CUDA device that is current for this rank.
    ShardedHead(const Tensor& W_shard, int row_offset, int total_rows, int rank, int world);
    ~ShardedHead();
    ShardedHead(const ShardedHead&) = delete;
    ShardedHead& operator=(const ShardedHead&) = delete;

    // Handle of this rank's exchange memory, to be sent to every other rank.
    IpcHandle local_handle() const { return handle_; }
    // All ranks' handles, indexed by rank (the own entry is ignored). Call once, on every rank.
    void connect(const std::vector<IpcHandle>& handles);

    // x: (in, 1) activations on this device (FP32 / FP16 / BF16). Enqueues the kernel on the
    // current stream. Every rank must call forward the same number of times.
    void forward(const Tensor& x, const Tensor* bias_shard = nullptr);
    // The same with another weight tensor of the shard's shape, dtype and device (e.g. the
    // benchmark's rotation over weight replicas that keeps the L2 cold).
    void forward_with(const Tensor& W_shard, const Tensor& x, const Tensor* bias_shard = nullptr);
    // Candidate form, k in 1..8: after the kernel, top_values() / top_rows() hold the k largest logits of
    // the WHOLE matrix (largest first, equal values: lower row first) and their rows, on every rank;
    // logits() is then complete for this rank's own rows only. May be mixed with forward().
    void forward_topk(const Tensor& x, int k, const Tensor* bias_shard = nullptr);
    void forward_topk_with(const Tensor& W_shard, const Tensor& x, int k, const Tensor* bias_shard = nullptr);
    const float* top_values() const;  // device pointers, 8 entries each, the first k valid
    const std::int32_t* top_rows() const;
    // Device pointer to the full result vector of the most recent forward (total_rows floats),
    // valid once that forward's kernel has completed on the stream.
    const float* logits() const;
    std::uint64_t calls() const { return calls_; }
    int total_rows() const { return total_rows_; }
    Device device() const { return W_->device; }

private:
    const Tensor* W_;
    int row_offset_, total_rows_, rank_, world_;
    void* local_ = nullptr;                  // exchange memory of this rank
    std::vector<void*> peer_base_;           // mapped exchange memory of every rank (own = local_)
    std::vector<void*> peer_out_, peer_cand_;
    void* state_ = nullptr;
    IpcHandle handle_{};
    std::uint64_t calls_ = 0;
    bool connected_ = false;
    static constexpr std::size_t kCandBytes = 2u * 8u * 256u * 8u * 8u;
    // two result vectors of floats and two vectors of 8-byte transfer words
    std::size_t out_bytes() const { return 24u * static_cast<std::size_t>(total_rows_); }
    void run(const Tensor& W, const Tensor& x, const Tensor* bias_shard, int k);
};

}  // namespace brotensor_b200

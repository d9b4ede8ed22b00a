// ShardedHead: exchange-memory set-up over CUDA IPC and the one-kernel forward.
#include "brotensor_b200/sharded_head.h"
#include "brotensor_b200/repack.h"

#include <cuda_runtime_api.h>

#include <cstring>
#include <stdexcept>
#include <string>

#include "b200q.h"
#include "brotensor_b200/runtime.h"

namespace brotensor_b200 {
namespace {
void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) {
        cudaGetLastError();
        throw std::runtime_error(std::string("brotensor: sharded_head: ") + what + ": " + cudaGetErrorString(e));
    }
}
int dt_code(Dtype d) {
    switch (d) {
        case Dtype::FP32: return B200Q_DT_F32;
        case Dtype::FP16: return B200Q_DT_F16;
        case Dtype::BF16: return B200Q_DT_BF16;
        default: throw std::runtime_error("brotensor: sharded_head: x must be FP32, FP16 or BF16");
    }
}
}  // namespace

ShardedHead::ShardedHead(const Tensor& W_shard, int row_offset, int total_rows, int rank, int world)
    : W_(&W_shard), row_offset_(row_offset), total_rows_(total_rows), rank_(rank), world_(world) {
    if (world < 1 || world > 8 || rank < 0 || rank >= world)
        throw std::runtime_error("brotensor: sharded_head: rank/world out of range (at most 8 ranks)");
    if (W_shard.device.type != DeviceType::CUDA) throw std::runtime_error("brotensor: sharded_head: W must be on a CUDA device");
    if (W_shard.dtype != Dtype::Q4_K && W_shard.dtype != Dtype::Q6_K && W_shard.dtype != Dtype::Q8_0)
        throw std::runtime_error("brotensor: sharded_head: W must be Q4_K, Q6_K or Q8_0");
    if (row_offset < 0 || W_shard.rows <= 0 || row_offset + W_shard.rows > total_rows)
        throw std::runtime_error("brotensor: sharded_head: shard rows do not lie inside the matrix");
    cuda_check(cudaSetDevice(W_shard.device.index), "cudaSetDevice");
    // exchange memory: [2][total_rows] floats (the result vectors), [2][total_rows] 8-byte transfer words
    // (b200q_gemv_shard), then the candidate table [2 parities][8 ranks][256 CTA slots][8] x 8 bytes
    // (b200q_gemv_shard_topk)
    const std::size_t bytes = out_bytes() + kCandBytes;
    cuda_check(cudaMalloc(&local_, bytes), "cudaMalloc(exchange memory)");
    cuda_check(cudaMemset(local_, 0, bytes), "cudaMemset");
    cuda_check(cudaMalloc(&state_, 256), "cudaMalloc(state)");
    cuda_check(cudaMemset(state_, 0, 256), "cudaMemset");
    cuda_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    cudaIpcMemHandle_t h;
    cuda_check(cudaIpcGetMemHandle(&h, local_), "cudaIpcGetMemHandle");
    static_assert(sizeof(h) == 64, "CUDA IPC handles are 64 bytes");
    std::memcpy(handle_.data(), &h, 64);
    peer_base_.assign(world, nullptr);
    peer_base_[rank] = local_;
    if (world == 1) connect({handle_});
}

void ShardedHead::connect(const std::vector<IpcHandle>& handles) {
    if (connected_) throw std::runtime_error("brotensor: sharded_head: connect called twice");
    if (static_cast<int>(handles.size()) != world_) throw std::runtime_error("brotensor: sharded_head: one handle per rank expected");
    cuda_check(cudaSetDevice(W_->device.index), "cudaSetDevice");
    for (int q = 0; q < world_; ++q) {
        if (q == rank_) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, handles[q].data(), 64);
        cuda_check(cudaIpcOpenMemHandle(&peer_base_[q], h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    }
    peer_out_.resize(world_);
    peer_cand_.resize(world_);
    for (int q = 0; q < world_; ++q) {
        peer_out_[q] = peer_base_[q];
        peer_cand_[q] = static_cast<char*>(peer_base_[q]) + out_bytes();
    }
    connected_ = true;
}

ShardedHead::~ShardedHead() {
    cudaSetDevice(W_->device.index);
    cudaDeviceSynchronize();
    for (int q = 0; q < world_; ++q)
        if (q != rank_ && peer_base_.size() > static_cast<std::size_t>(q) && peer_base_[q]) cudaIpcCloseMemHandle(peer_base_[q]);
    if (local_) cudaFree(local_);
    if (state_) cudaFree(state_);
    cudaGetLastError();
}

void ShardedHead::forward(const Tensor& x, const Tensor* bias_shard) { run(*W_, x, bias_shard, 0); }
void ShardedHead::forward_with(const Tensor& W, const Tensor& x, const Tensor* bias_shard) { run(W, x, bias_shard, 0); }
void ShardedHead::forward_topk(const Tensor& x, int k, const Tensor* bias_shard) { forward_topk_with(*W_, x, k, bias_shard); }
void ShardedHead::forward_topk_with(const Tensor& W, const Tensor& x, int k, const Tensor* bias_shard) {
    if (k < 1 || k > 8) throw std::runtime_error("brotensor: sharded_head: k must be 1..8");
    run(W, x, bias_shard, k);
}

void ShardedHead::run(const Tensor& W, const Tensor& x, const Tensor* bias_shard, int k) {
    if (W.dtype != W_->dtype || W.rows != W_->rows || W.cols != W_->cols || W.device != W_->device)
        throw std::runtime_error("brotensor: sharded_head: weight does not match the shard this head was made for");
    if (!connected_) throw std::runtime_error("brotensor: sharded_head: forward before connect");
    if (x.device != W_->device) throw std::runtime_error("brotensor: sharded_head: x is on another device than W");
    if (x.rows != W_->cols || x.cols != 1) throw std::runtime_error("brotensor: sharded_head: x must be (in, 1)");
    if (bias_shard && (bias_shard->dtype != x.dtype || bias_shard->rows * bias_shard->cols != W_->rows))
        throw std::runtime_error("brotensor: sharded_head: bias must hold this shard's rows in x's dtype");
    cuda_check(cudaSetDevice(W_->device.index), "cudaSetDevice");
    const int wfmt = (W.dtype == Dtype::Q6_K && is_repacked(W)) ? B200Q_FMT_Q6_K_R8 : static_cast<int>(W.dtype);
    const void* b = bias_shard ? bias_shard->data : nullptr;
    // this rank's results of the candidate form live behind the two state words
    char* st = static_cast<char*>(state_);
    const int rc = k == 0 ? b200q_gemv_shard(wfmt, W.data, x.data, dt_code(x.dtype), b, W_->rows, W_->cols, row_offset_, total_rows_, rank_,
                                             world_, peer_out_.data(), state_, cuda_current_stream())
                          : b200q_gemv_shard_topk(wfmt, W.data, x.data, dt_code(x.dtype), b, W_->rows, W_->cols, row_offset_, total_rows_,
                                                  rank_, world_, peer_out_.data(), peer_cand_.data(), state_, k,
                                                  st + 64, st + 128, cuda_current_stream());
    if (rc != B200Q_OK) throw std::runtime_error(std::string("brotensor: sharded_head: ") + b200q_last_error());
    ++calls_;
}

const float* ShardedHead::top_values() const { return reinterpret_cast<const float*>(static_cast<const char*>(state_) + 64); }
const std::int32_t* ShardedHead::top_rows() const { return reinterpret_cast<const std::int32_t*>(static_cast<const char*>(state_) + 128); }

const float* ShardedHead::logits() const {
    return static_cast<const float*>(local_) + (calls_ & 1u) * static_cast<std::size_t>(total_rows_);
}

}  // namespace brotensor_b200

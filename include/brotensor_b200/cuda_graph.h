// CUDA graph capture / replay of a fixed-shape op sequence, e.g. the GEMVs of one decode
// step with their host round trips: capture once, then one launch per step instead of one
// per kernel and copy. Mirrors include/brotensor/cuda_graph.h:44-90 (same classes, same
// contract): warm up once so every output is allocated, capture an identical run that
// reuses those tensors, feed new inputs by writing into the same buffers, launch, sync.
#pragma once

#include <memory>

namespace brotensor_b200 {

// An instantiated, replayable graph. Move-only.
class CudaGraph {
public:
    CudaGraph();
    ~CudaGraph();
    CudaGraph(CudaGraph&&) noexcept;
    CudaGraph& operator=(CudaGraph&&) noexcept;
    CudaGraph(const CudaGraph&) = delete;
    CudaGraph& operator=(const CudaGraph&) = delete;

    bool valid() const;
    // Replays the captured sequence on the calling thread's current stream; does not
    // synchronise. Throws if the handle is empty.
    void launch();
    void reset();

private:
    struct Impl;
    std::unique_ptr<Impl> impl_;
    friend class CudaGraphCapture;
};

// RAII capture scope: creates a capture stream, makes it the calling thread's current
// stream and begins capture; finish() ends capture, instantiates and restores the previous
// stream. Destroyed without finish(), the capture is abandoned and the stream restored.
class CudaGraphCapture {
public:
    CudaGraphCapture();
    ~CudaGraphCapture();
    CudaGraphCapture(const CudaGraphCapture&) = delete;
    CudaGraphCapture& operator=(const CudaGraphCapture&) = delete;
    CudaGraph finish();

private:
    struct Impl;
    std::unique_ptr<Impl> impl_;
};

}  // namespace brotensor_b200

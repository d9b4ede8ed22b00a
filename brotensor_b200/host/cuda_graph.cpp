// CudaGraph / CudaGraphCapture over the CUDA runtime's stream capture.
#include "brotensor_b200/cuda_graph.h"

#include <cuda_runtime_api.h>

#include <stdexcept>
#include <string>

#include "brotensor_b200/runtime.h"

namespace brotensor_b200 {
namespace {
void check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) {
        cudaGetLastError();
        throw std::runtime_error(std::string("brotensor: cuda_graph: ") + what + ": " + cudaGetErrorString(e));
    }
}
}  // namespace

struct CudaGraph::Impl {
    cudaGraphExec_t exec = nullptr;
};

CudaGraph::CudaGraph() : impl_(new Impl) {}
CudaGraph::~CudaGraph() { reset(); }
CudaGraph::CudaGraph(CudaGraph&& o) noexcept : impl_(std::move(o.impl_)) { o.impl_.reset(new Impl); }
CudaGraph& CudaGraph::operator=(CudaGraph&& o) noexcept {
    if (this != &o) {
        reset();
        impl_ = std::move(o.impl_);
        o.impl_.reset(new Impl);
    }
    return *this;
}
bool CudaGraph::valid() const { return impl_ && impl_->exec != nullptr; }
void CudaGraph::reset() {
    if (impl_ && impl_->exec) {
        cudaGraphExecDestroy(impl_->exec);
        impl_->exec = nullptr;
    }
}
void CudaGraph::launch() {
    if (!valid()) throw std::runtime_error("brotensor: CudaGraph::launch: no captured graph");
    check(cudaGraphLaunch(impl_->exec, static_cast<cudaStream_t>(cuda_current_stream())), "cudaGraphLaunch");
}

struct CudaGraphCapture::Impl {
    cudaStream_t stream = nullptr;
    void* prev = nullptr;
    bool capturing = false;
};

CudaGraphCapture::CudaGraphCapture() : impl_(new Impl) {
    // Thread-local capture mode: other threads may keep using the legacy stream meanwhile.
    check(cudaStreamCreateWithFlags(&impl_->stream, cudaStreamNonBlocking), "cudaStreamCreateWithFlags");
    impl_->prev = cuda_current_stream();
    cuda_set_stream(impl_->stream);
    const cudaError_t e = cudaStreamBeginCapture(impl_->stream, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) {
        cuda_set_stream(impl_->prev);
        cudaStreamDestroy(impl_->stream);
        impl_->stream = nullptr;
        check(e, "cudaStreamBeginCapture");
    }
    impl_->capturing = true;
}

CudaGraph CudaGraphCapture::finish() {
    if (!impl_->capturing) throw std::runtime_error("brotensor: CudaGraphCapture::finish: not capturing");
    cudaGraph_t graph = nullptr;
    impl_->capturing = false;
    const cudaError_t e = cudaStreamEndCapture(impl_->stream, &graph);
    cuda_set_stream(impl_->prev);
    check(e, "cudaStreamEndCapture");
    CudaGraph g;
    const cudaError_t e2 = cudaGraphInstantiate(&g.impl_->exec, graph, 0);
    cudaGraphDestroy(graph);
    check(e2, "cudaGraphInstantiate");
    return g;
}

CudaGraphCapture::~CudaGraphCapture() {
    if (impl_->capturing) {  // abandoned: end the capture, drop what was recorded
        cudaGraph_t graph = nullptr;
        cudaStreamEndCapture(impl_->stream, &graph);
        if (graph) cudaGraphDestroy(graph);
        cuda_set_stream(impl_->prev);
        cudaGetLastError();
    }
    if (impl_->stream) cudaStreamDestroy(impl_->stream);
}

}  // namespace brotensor_b200

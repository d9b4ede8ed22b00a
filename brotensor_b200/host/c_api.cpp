// Flat C entry points over the C++ host layer, for callers without a C++ toolchain
// (the Python tests and the benchmark's end-to-end arm bind them with ctypes). They add
// no behaviour: every call goes through Tensor / the dispatcher / the public ops, so what
// is measured or tested through them is the plugin path a C++ user takes.
#include <cstring>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "brotensor_b200/cuda_graph.h"
#include "brotensor_b200/gguf.h"
#include "brotensor_b200/ops/quant.h"
#include "brotensor_b200/runtime.h"
#include "brotensor_b200/repack.h"
#include "brotensor_b200/sharded_head.h"

using namespace brotensor_b200;

namespace {
thread_local std::string t_err;
template <typename F>
int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        t_err = e.what();
        return -1;
    }
}
Dtype fmt_dtype(int fmt) { return static_cast<Dtype>(fmt); }

struct Session {
    const Tensor* W;
    Tensor x, y, bias;
    bool has_bias = false;
    int M;
};
}  // namespace

extern "C" {

const char* b200h_last_error() { return t_err.c_str(); }

// Brings the backends up; returns the number of CUDA devices (0 on a CPU-only host).
int b200h_init() {
    if (guarded([] { init(); })) return -1;
    return cuda_device_count();
}

// The calling thread's stream for ops on device `dev` (a cudaStream_t; NULL = legacy default stream).
void b200h_set_stream(void* stream, int dev) { cuda_set_stream(stream, dev); }

// ---- weights -----------------------------------------------------------------------------
// `device` < 0 keeps the tensor on the host. Returns an owning handle or NULL.
void* b200h_weight_from_host(int fmt, const void* bytes, int rows, int cols, int device) {
    Tensor* t = nullptr;
    if (guarded([&] {
            const Device d = device < 0 ? Device::CPU : Device::cuda(device);
            const Dtype dt = fmt_dtype(fmt);
            t = new Tensor(Tensor::from_raw_bytes_on(d, bytes, rows, cols, dt,
                                                     dtype_storage_bytes(dt, static_cast<std::int64_t>(rows) * cols)));
        }))
        return nullptr;
    return t;
}
// Non-owning Tensor over quantized blocks already resident on `device` (freed by its owner).
void* b200h_weight_view(int fmt, void* dev_bytes, int rows, int cols, int device) {
    Tensor* t = nullptr;
    if (guarded([&] { t = new Tensor(Tensor::view(Device::cuda(device), dev_bytes, rows, cols, fmt_dtype(fmt))); })) return nullptr;
    return t;
}
void b200h_tensor_free(void* t) { delete static_cast<Tensor*>(t); }
// repack_weights / unpack_weights / is_repacked on a weight handle (include/brotensor_b200/repack.h).
// b200h_weight_repack returns 1 when the weight is in the regrouped layout afterwards, 0 when its
// format has none, -1 on error.
int b200h_weight_repack(void* t) {
    int r = 0;
    if (guarded([&] { r = repack_weights(*static_cast<Tensor*>(t)) ? 1 : 0; })) return -1;
    return r;
}
int b200h_weight_unpack(void* t) {
    return guarded([&] { unpack_weights(*static_cast<Tensor*>(t)); });
}
int b200h_weight_is_repacked(void* t) { return is_repacked(*static_cast<Tensor*>(t)) ? 1 : 0; }
void* b200h_tensor_data(void* t) { return static_cast<Tensor*>(t)->data; }
int b200h_tensor_rows(void* t) { return static_cast<Tensor*>(t)->rows; }
int b200h_tensor_cols(void* t) { return static_cast<Tensor*>(t)->cols; }
int b200h_tensor_dtype(void* t) { return static_cast<int>(static_cast<Tensor*>(t)->dtype); }
int b200h_tensor_to_host(void* t, void* dst) {
    return guarded([&] { static_cast<Tensor*>(t)->copy_raw_to_host(dst); });
}

// ---- ops through the public signatures -----------------------------------------------------
// dequant_*_to_fp16: out_dtype 1 (FP16, the reference behaviour), 0 (FP32) or 4 (BF16).
int b200h_dequant(void* Wh, void* out_host, int out_dtype) {
    return guarded([&] {
        const Tensor& W = *static_cast<Tensor*>(Wh);
        Tensor out;
        if (out_dtype != 1) out = Tensor::empty_on(W.device, W.rows, W.cols, static_cast<Dtype>(out_dtype));
        switch (W.dtype) {
            case Dtype::Q4_K: dequant_q4k_to_fp16(W, out); break;
            case Dtype::Q6_K: dequant_q6k_to_fp16(W, out); break;
            case Dtype::Q8_0: dequant_q8_0_to_fp16(W, out); break;
            default: throw std::runtime_error("b200h_dequant: weight is not Q4_K / Q6_K / Q8_0");
        }
        sync(W.device);
        out.copy_raw_to_host(out_host);
    });
}

// A session keeps the device-side activation and result tensors of one linear layer, so
// a step is: host -> device copy of X, the op, device -> host copy of Y.
void* b200h_session_create(void* Wh, int M, int x_dtype, int y_dtype, const void* bias_host) {
    Session* s = nullptr;
    if (guarded([&] {
            const Tensor& W = *static_cast<Tensor*>(Wh);
            auto up = std::make_unique<Session>();
            up->W = &W;
            up->M = M;
            const Dtype xd = static_cast<Dtype>(x_dtype), yd = static_cast<Dtype>(y_dtype);
            if (M == 1) {
                up->x = Tensor::empty_on(W.device, W.cols, 1, xd);
                up->y = Tensor::empty_on(W.device, W.rows, 1, yd);
            } else {
                up->x = Tensor::empty_on(W.device, M, W.cols, xd);
                up->y = Tensor::empty_on(W.device, M, W.rows, yd);
            }
            if (bias_host) {
                up->bias = Tensor::from_raw_bytes_on(W.device, bias_host, W.rows, 1, xd, dtype_storage_bytes(xd, W.rows));
                up->has_bias = true;
            }
            s = up.release();
        }))
        return nullptr;
    return s;
}
void b200h_session_free(void* s) { delete static_cast<Session*>(s); }

int b200h_session_run(void* sh, const void* x_host, void* y_host) {
    return guarded([&] {
        Session& s = *static_cast<Session*>(sh);
        const Tensor& W = *s.W;
        // the same copies Tensor::from_raw_bytes_on / copy_to_host make, into resident tensors
        Tensor xin = Tensor::from_raw_bytes_on(Device::CPU, x_host, s.x.rows, s.x.cols, s.x.dtype, s.x.bytes());
        Tensor xdev = xin.to(W.device);
        const Tensor* b = s.has_bias ? &s.bias : nullptr;
        const bool gemv = s.M == 1;
        switch (W.dtype) {
            case Dtype::Q4_K: gemv ? linear_forward_q4k_fp16(W, b, xdev, s.y) : linear_forward_batched_q4k_fp16(W, b, xdev, s.y); break;
            case Dtype::Q6_K: gemv ? linear_forward_q6k_fp16(W, b, xdev, s.y) : linear_forward_batched_q6k_fp16(W, b, xdev, s.y); break;
            case Dtype::Q8_0: gemv ? linear_forward_q8_0_fp16(W, b, xdev, s.y) : linear_forward_batched_q8_0_fp16(W, b, xdev, s.y); break;
            default: throw std::runtime_error("b200h_session_run: weight is not Q4_K / Q6_K / Q8_0");
        }
        s.y.copy_raw_to_host(y_host);
    });
}
// The same step without blocking: x_pinned and y_pinned are page-locked host buffers; the copy
// in, the op and the copy out are enqueued on the calling thread's stream. b200h_sync() makes
// y_pinned valid. Several sessions may be enqueued before one sync.
int b200h_session_enqueue(void* sh, const void* x_pinned, void* y_pinned) {
    return guarded([&] {
        Session& s = *static_cast<Session*>(sh);
        const Tensor& W = *s.W;
        s.x.copy_raw_from_host_async(x_pinned);
        const Tensor* b = s.has_bias ? &s.bias : nullptr;
        const bool gemv = s.M == 1;
        switch (W.dtype) {
            case Dtype::Q4_K: gemv ? linear_forward_q4k_fp16(W, b, s.x, s.y) : linear_forward_batched_q4k_fp16(W, b, s.x, s.y); break;
            case Dtype::Q6_K: gemv ? linear_forward_q6k_fp16(W, b, s.x, s.y) : linear_forward_batched_q6k_fp16(W, b, s.x, s.y); break;
            case Dtype::Q8_0: gemv ? linear_forward_q8_0_fp16(W, b, s.x, s.y) : linear_forward_batched_q8_0_fp16(W, b, s.x, s.y); break;
            default: throw std::runtime_error("b200h_session_enqueue: weight is not Q4_K / Q6_K / Q8_0");
        }
        s.y.copy_raw_to_host_async(y_pinned);
    });
}
// ---- a set of GEMV layers whose activations and results live in one device arena each, so a
// step's host round trip is ONE copy in and ONE copy out around the ops (what a decode loop
// does: a layer's activations sit in one buffer). x/y of op i are views into the arenas.
struct LayerSet {
    std::vector<const Tensor*> W;
    Tensor X_all, Y_all;
    std::vector<Tensor> x, y;
    std::vector<unsigned long long> x_off, y_off;
    unsigned long long x_bytes = 0, y_bytes = 0;
};
void* b200h_layer_create(void* const* weights, int n, int x_dtype, int y_dtype) {
    LayerSet* L = nullptr;
    if (guarded([&] {
            auto up = std::make_unique<LayerSet>();
            const Dtype xd = static_cast<Dtype>(x_dtype), yd = static_cast<Dtype>(y_dtype);
            if (n <= 0) throw std::runtime_error("b200h_layer_create: no layers");
            const Device dev = static_cast<const Tensor*>(weights[0])->device;
            auto pad = [](unsigned long long v) { return (v + 255ull) & ~255ull; };
            for (int i = 0; i < n; ++i) {
                const Tensor* W = static_cast<const Tensor*>(weights[i]);
                if (W->device != dev) throw std::runtime_error("b200h_layer_create: weights on different devices");
                up->W.push_back(W);
                up->x_off.push_back(up->x_bytes);
                up->y_off.push_back(up->y_bytes);
                up->x_bytes += pad(dtype_storage_bytes(xd, W->cols));
                up->y_bytes += pad(dtype_storage_bytes(yd, W->rows));
            }
            up->X_all = Tensor::zeros_on(dev, static_cast<int>(up->x_bytes / 4), 1, Dtype::FP32);
            up->Y_all = Tensor::zeros_on(dev, static_cast<int>(up->y_bytes / 4), 1, Dtype::FP32);
            for (int i = 0; i < n; ++i) {
                up->x.push_back(Tensor::view(dev, static_cast<char*>(up->X_all.data) + up->x_off[i], up->W[i]->cols, 1, xd));
                up->y.push_back(Tensor::view(dev, static_cast<char*>(up->Y_all.data) + up->y_off[i], up->W[i]->rows, 1, yd));
            }
            L = up.release();
        }))
        return nullptr;
    return L;
}
void b200h_layer_free(void* h) { delete static_cast<LayerSet*>(h); }
// Byte offsets of every op's x and y inside the arenas (the host arenas use the same layout).
int b200h_layer_layout(void* h, unsigned long long* x_off, unsigned long long* y_off, unsigned long long* x_bytes,
                       unsigned long long* y_bytes) {
    LayerSet& L = *static_cast<LayerSet*>(h);
    for (std::size_t i = 0; i < L.W.size(); ++i) {
        x_off[i] = L.x_off[i];
        y_off[i] = L.y_off[i];
    }
    *x_bytes = L.x_bytes;
    *y_bytes = L.y_bytes;
    return 0;
}
// One copy in (page-locked x arena), the n GEMVs through the public ops, one copy out.
int b200h_layer_enqueue(void* h, const void* x_pinned_arena, void* y_pinned_arena) {
    return guarded([&] {
        LayerSet& L = *static_cast<LayerSet*>(h);
        L.X_all.copy_raw_from_host_async(x_pinned_arena);
        for (std::size_t i = 0; i < L.W.size(); ++i) {
            const Tensor& W = *L.W[i];
            switch (W.dtype) {
                case Dtype::Q4_K: linear_forward_q4k_fp16(W, nullptr, L.x[i], L.y[i]); break;
                case Dtype::Q6_K: linear_forward_q6k_fp16(W, nullptr, L.x[i], L.y[i]); break;
                case Dtype::Q8_0: linear_forward_q8_0_fp16(W, nullptr, L.x[i], L.y[i]); break;
                default: throw std::runtime_error("b200h_layer_enqueue: weight is not Q4_K / Q6_K / Q8_0");
            }
        }
        L.Y_all.copy_raw_to_host_async(y_pinned_arena);
    });
}

// ---- graph capture of a sequence of the calls above (CudaGraphCapture / CudaGraph) -------------
void* b200h_capture_begin() {
    CudaGraphCapture* c = nullptr;
    if (guarded([&] { c = new CudaGraphCapture(); })) return nullptr;
    return c;
}
// Ends the capture (consumes the capture handle) and returns a graph handle, or NULL.
void* b200h_capture_finish(void* ch) {
    std::unique_ptr<CudaGraphCapture> c(static_cast<CudaGraphCapture*>(ch));
    CudaGraph* g = nullptr;
    if (guarded([&] { g = new CudaGraph(c->finish()); })) return nullptr;
    return g;
}
int b200h_graph_launch(void* gh) {
    return guarded([&] { static_cast<CudaGraph*>(gh)->launch(); });
}
void b200h_graph_free(void* gh) { delete static_cast<CudaGraph*>(gh); }

int b200h_sync(int device) {
    return guarded([&] { sync(device < 0 ? Device::CPU : Device::cuda(device)); });
}
int b200h_session_y_dtype(void* sh) { return static_cast<int>(static_cast<Session*>(sh)->y.dtype); }

// ---- row-sharded LM head -----------------------------------------------------------------------
// create -> exchange the 64-byte handles between the ranks -> connect -> run ... -> free
void* b200h_head_create(void* W_shard, int row_offset, int total_rows, int rank, int world, unsigned char* handle64) {
    ShardedHead* h = nullptr;
    if (guarded([&] {
            h = new ShardedHead(*static_cast<Tensor*>(W_shard), row_offset, total_rows, rank, world);
            const IpcHandle hd = h->local_handle();
            std::memcpy(handle64, hd.data(), 64);
        }))
        return nullptr;
    return h;
}
int b200h_head_connect(void* hh, const unsigned char* handles, int world) {
    return guarded([&] {
        std::vector<IpcHandle> v(world);
        for (int q = 0; q < world; ++q) std::memcpy(v[q].data(), handles + 64 * q, 64);
        static_cast<ShardedHead*>(hh)->connect(v);
    });
}
// x_dev: device pointer to `in` values of x_dtype on the head's device (already resident: the
// decode loop keeps activations on the device between layers).
int b200h_head_run(void* hh, void* W_or_null, void* x_dev, int in, int x_dtype) {
    return guarded([&] {
        ShardedHead& h = *static_cast<ShardedHead*>(hh);
        const Tensor x = Tensor::view(h.device(), x_dev, in, 1, static_cast<Dtype>(x_dtype));
        if (W_or_null) h.forward_with(*static_cast<Tensor*>(W_or_null), x);
        else h.forward(x);
    });
}
// The candidate form: k (value, row) pairs instead of the logits cross the links.
int b200h_head_run_topk(void* hh, void* W_or_null, void* x_dev, int in, int x_dtype, int k) {
    return guarded([&] {
        ShardedHead& h = *static_cast<ShardedHead*>(hh);
        const Tensor x = Tensor::view(h.device(), x_dev, in, 1, static_cast<Dtype>(x_dtype));
        if (W_or_null) h.forward_topk_with(*static_cast<Tensor*>(W_or_null), x, k);
        else h.forward_topk(x, k);
    });
}
// Waits for the head's device, then copies the k candidates of the latest run_topk (values, rows).
int b200h_head_top_to_host(void* hh, float* vals, int* rows, int k) {
    return guarded([&] {
        ShardedHead& h = *static_cast<ShardedHead*>(hh);
        sync(h.device());
        Tensor::view(h.device(), const_cast<float*>(h.top_values()), k, 1, Dtype::FP32).copy_to_host(vals);
        Tensor::view(h.device(), const_cast<std::int32_t*>(h.top_rows()), k, 1, Dtype::INT32).copy_raw_to_host(rows);
    });
}
const void* b200h_head_top_rows(void* hh) { return static_cast<ShardedHead*>(hh)->top_rows(); }
// Waits for the head's device, then copies the latest full result vector to `dst` (total_rows floats).
int b200h_head_logits_to_host(void* hh, float* dst) {
    return guarded([&] {
        ShardedHead& h = *static_cast<ShardedHead*>(hh);
        sync(h.device());
        const Tensor v = Tensor::view(h.device(), const_cast<float*>(h.logits()), h.total_rows(), 1, Dtype::FP32);
        v.copy_to_host(dst);
    });
}
const void* b200h_head_logits(void* hh) { return static_cast<ShardedHead*>(hh)->logits(); }
unsigned long long b200h_head_calls(void* hh) { return static_cast<ShardedHead*>(hh)->calls(); }
void b200h_head_free(void* hh) { delete static_cast<ShardedHead*>(hh); }

// ---- GGUF ------------------------------------------------------------------------------------
void* b200h_gguf_open(const char* path) {
    gguf::File* f = nullptr;
    if (guarded([&] { f = new gguf::File(gguf::File::open(path)); })) return nullptr;
    return f;
}
void b200h_gguf_close(void* f) { delete static_cast<gguf::File*>(f); }
int b200h_gguf_tensor_count(void* f) { return static_cast<int>(static_cast<gguf::File*>(f)->tensor_count()); }
unsigned b200h_gguf_alignment(void* f) { return static_cast<gguf::File*>(f)->alignment(); }
unsigned b200h_gguf_version(void* f) { return static_cast<gguf::File*>(f)->version(); }
int b200h_gguf_meta_count(void* f) { return static_cast<int>(static_cast<gguf::File*>(f)->metadata().size()); }
// Value of a metadata key rendered as text (scalars and strings; arrays as their length).
int b200h_gguf_meta_text(void* fh, const char* key, char* out, int cap) {
    return guarded([&] {
        const gguf::Value& v = static_cast<gguf::File*>(fh)->get_meta(key);
        std::string s;
        using VT = gguf::ValueType;
        switch (v.type) {
            case VT::U8: s = std::to_string(v.scalar.u8); break;
            case VT::I8: s = std::to_string(v.scalar.i8); break;
            case VT::U16: s = std::to_string(v.scalar.u16); break;
            case VT::I16: s = std::to_string(v.scalar.i16); break;
            case VT::U32: s = std::to_string(v.scalar.u32); break;
            case VT::I32: s = std::to_string(v.scalar.i32); break;
            case VT::U64: s = std::to_string(v.scalar.u64); break;
            case VT::I64: s = std::to_string(v.scalar.i64); break;
            case VT::F32: s = std::to_string(v.scalar.f32); break;
            case VT::F64: s = std::to_string(v.scalar.f64); break;
            case VT::Bool: s = v.scalar.b ? "true" : "false"; break;
            case VT::String: s = v.str; break;
            case VT::Array: s = "array[" + std::to_string(v.array.size()) + "]"; break;
        }
        std::strncpy(out, s.c_str(), cap - 1);
        out[cap - 1] = 0;
    });
}
int b200h_gguf_tensor(void* fh, int i, char* name, int namelen, long long* shape8, int* ndims, unsigned* ggml_type,
                      int* dtype, int* supported, unsigned long long* nbytes, long long* numel,
                      unsigned long long* data_off_from_first) {
    return guarded([&] {
        const auto& ts = static_cast<gguf::File*>(fh)->tensors();
        if (i < 0 || i >= static_cast<int>(ts.size())) throw std::runtime_error("gguf: tensor index out of range");
        const gguf::TensorInfo& t = ts[i];
        std::strncpy(name, t.name.c_str(), namelen - 1);
        name[namelen - 1] = 0;
        *ndims = static_cast<int>(t.shape.size());
        for (int d = 0; d < *ndims && d < 8; ++d) shape8[d] = t.shape[d];
        *ggml_type = t.ggml_type;
        *dtype = static_cast<int>(t.dtype);
        *supported = t.dtype_supported ? 1 : 0;
        *nbytes = t.nbytes;
        *numel = t.numel;
        *data_off_from_first = static_cast<unsigned long long>(t.data - ts[0].data);
    });
}
int b200h_shape_to_2d(const long long* shape, int n, int* rows, int* cols) {
    return guarded([&] {
        std::vector<std::int64_t> s(shape, shape + n);
        auto rc = gguf::shape_to_2d(s);
        *rows = rc.first;
        *cols = rc.second;
    });
}
// Rows [row_begin, row_end) of tensor i as (rows, cols) on `device` (< 0: host). NULL on error.
void* b200h_gguf_upload_rows(void* fh, int i, int rows, int cols, int row_begin, int row_end, int device) {
    Tensor* t = nullptr;
    if (guarded([&] {
            const auto& ts = static_cast<gguf::File*>(fh)->tensors();
            if (i < 0 || i >= static_cast<int>(ts.size())) throw std::runtime_error("gguf: tensor index out of range");
            auto up = std::make_unique<Tensor>();
            gguf::upload_rows(ts[i], rows, cols, row_begin, row_end, device < 0 ? Device::CPU : Device::cuda(device), *up);
            t = up.release();
        }))
        return nullptr;
    return t;
}

}  // extern "C"

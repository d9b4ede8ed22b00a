// mmap'd GGUF reader (versions 2 and 3) and the device upload path.
//
// Reading contract and error cases follow brotensor's loader (src/gguf.cpp:111-130 type
// table, :134-191 bounds-checked reader, :246-263 shape_to_2d, :317-445 File::open,
// :473-500 upload_raw); all failures are std::runtime_error("gguf: <reason>").
// The upload differs: instead of one blocking cudaMemcpy from the pageable mapping
// (src/cuda/tensor.cu:134-142) the bytes go through two pinned staging buffers with
// asynchronous copies, so reading the file overlaps the transfer, and a contiguous row
// range of a tensor can be uploaded on its own (the shard of a row-sharded weight).
#include "brotensor_b200/gguf.h"
#include "brotensor_b200/repack.h"

#include <cuda_runtime_api.h>

#include <mutex>
#include <thread>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <climits>
#include <cstdlib>
#include <cstring>
#include <stdexcept>

#include "brotensor_b200/runtime.h"

namespace brotensor_b200::gguf {

namespace {

[[noreturn]] void fail(const std::string& msg) { throw std::runtime_error("gguf: " + msg); }

struct TypeRow {
    Dtype dtype;
    bool supported;
    int block, bytes;
};
TypeRow type_row(std::uint32_t t) {
    switch (t) {
        case 0: return {Dtype::FP32, true, 1, 4};
        case 1: return {Dtype::FP16, true, 1, 2};
        case 2: return {Dtype::Q4_0, true, 32, 18};
        case 3: return {Dtype::Q4_1, true, 32, 20};
        case 6: return {Dtype::Q5_0, true, 32, 22};
        case 7: return {Dtype::Q5_1, true, 32, 24};
        case 8: return {Dtype::Q8_0, true, 32, 34};
        case 9: return {Dtype::Q8_1, true, 32, 36};
        case 10: return {Dtype::Q2_K, true, 256, 82};
        case 11: return {Dtype::Q3_K, true, 256, 110};
        case 12: return {Dtype::Q4_K, true, 256, 144};
        case 13: return {Dtype::Q5_K, true, 256, 176};
        case 14: return {Dtype::Q6_K, true, 256, 210};
        case 15: return {Dtype::Q8_K, true, 256, 292};
        case 30: return {Dtype::BF16, true, 1, 2};
        default: return {Dtype::FP32, false, 0, 0};
    }
}

// Cursor over the mapping. `pos <= size` always holds, so `n > size - pos` cannot wrap
// even for lengths read straight off a hostile file.
struct Cursor {
    const std::uint8_t* base;
    std::size_t pos, size;
    void need(std::size_t n) const {
        if (n > size - pos) fail("unexpected EOF");
    }
    template <typename T>
    T get() {
        need(sizeof(T));
        T v;
        std::memcpy(&v, base + pos, sizeof(T));
        pos += sizeof(T);
        return v;
    }
    std::string str() {
        const std::uint64_t len = get<std::uint64_t>();
        if (len > size - pos) fail("unexpected EOF");
        std::string s(reinterpret_cast<const char*>(base + pos), static_cast<std::size_t>(len));
        pos += static_cast<std::size_t>(len);
        return s;
    }
};

Value read_value(Cursor& c, ValueType t) {
    Value v;
    v.type = t;
    switch (t) {
        case ValueType::U8: v.scalar.u8 = c.get<std::uint8_t>(); break;
        case ValueType::I8: v.scalar.i8 = c.get<std::int8_t>(); break;
        case ValueType::U16: v.scalar.u16 = c.get<std::uint16_t>(); break;
        case ValueType::I16: v.scalar.i16 = c.get<std::int16_t>(); break;
        case ValueType::U32: v.scalar.u32 = c.get<std::uint32_t>(); break;
        case ValueType::I32: v.scalar.i32 = c.get<std::int32_t>(); break;
        case ValueType::F32: v.scalar.f32 = c.get<float>(); break;
        case ValueType::U64: v.scalar.u64 = c.get<std::uint64_t>(); break;
        case ValueType::I64: v.scalar.i64 = c.get<std::int64_t>(); break;
        case ValueType::F64: v.scalar.f64 = c.get<double>(); break;
        case ValueType::Bool: {
            const std::uint8_t b = c.get<std::uint8_t>();
            if (b > 1) fail("bool value not 0 or 1");
            v.scalar.b = b != 0;
            break;
        }
        case ValueType::String: v.str = c.str(); break;
        case ValueType::Array: {
            const std::uint32_t et = c.get<std::uint32_t>();
            if (et > 12) fail("array element type out of range");
            v.array_elem_type = static_cast<ValueType>(et);
            const std::uint64_t len = c.get<std::uint64_t>();
            // every element takes at least one byte, so a length beyond the rest of the
            // file is corrupt; checking first keeps reserve() from a hostile allocation
            if (len > c.size - c.pos) fail("unexpected EOF");
            v.array.reserve(static_cast<std::size_t>(len));
            for (std::uint64_t i = 0; i < len; ++i) v.array.push_back(read_value(c, v.array_elem_type));
            break;
        }
    }
    return v;
}

}  // namespace

// ---- File ------------------------------------------------------------------------------

File::~File() { release_(); }

void File::release_() noexcept {
    if (base_) ::munmap(base_, size_);
    if (fd_ >= 0) ::close(fd_);
    base_ = nullptr;
    fd_ = -1;
    size_ = 0;
    version_ = 0;
    alignment_ = 32;
    metadata_.clear();
    meta_index_.clear();
    tensors_.clear();
    tensor_index_.clear();
}

File::File(File&& o) noexcept { *this = std::move(o); }

File& File::operator=(File&& o) noexcept {
    if (this != &o) {
        release_();
        fd_ = o.fd_; base_ = o.base_; size_ = o.size_;
        version_ = o.version_; alignment_ = o.alignment_;
        metadata_ = std::move(o.metadata_);
        meta_index_ = std::move(o.meta_index_);
        tensors_ = std::move(o.tensors_);
        tensor_index_ = std::move(o.tensor_index_);
        o.fd_ = -1; o.base_ = nullptr; o.size_ = 0; o.version_ = 0; o.alignment_ = 32;
        o.metadata_.clear(); o.meta_index_.clear(); o.tensors_.clear(); o.tensor_index_.clear();
    }
    return *this;
}

File File::open(const std::string& path) {
    File f;
    f.fd_ = ::open(path.c_str(), O_RDONLY);
    if (f.fd_ < 0) fail("cannot open '" + path + "'");
    struct stat st;
    if (::fstat(f.fd_, &st) != 0) fail("cannot stat '" + path + "'");
    if (st.st_size < 24) fail("file too small: '" + path + "'");
    f.size_ = static_cast<std::size_t>(st.st_size);
    void* m = ::mmap(nullptr, f.size_, PROT_READ, MAP_PRIVATE, f.fd_, 0);
    if (m == MAP_FAILED) {
        f.size_ = 0;
        fail("cannot map '" + path + "'");
    }
    f.base_ = m;  // from here on f's destructor unmaps on throw

    Cursor c{static_cast<const std::uint8_t*>(m), 0, f.size_};
    if (c.get<std::uint32_t>() != 0x46554747u) fail("bad magic (not a GGUF file)");
    const std::uint32_t version = c.get<std::uint32_t>();
    if (version != 2 && version != 3) fail("unsupported GGUF version " + std::to_string(version));
    f.version_ = version;
    const std::uint64_t n_tensors = c.get<std::uint64_t>();
    const std::uint64_t n_meta = c.get<std::uint64_t>();
    if (n_meta > f.size_ || n_tensors > f.size_) fail("unexpected EOF");

    for (std::uint64_t i = 0; i < n_meta; ++i) {
        std::string key = c.str();
        const std::uint32_t vt = c.get<std::uint32_t>();
        if (vt > 12) fail("metadata value type out of range");
        Value v = read_value(c, static_cast<ValueType>(vt));
        if (key == "general.alignment") {
            if (v.type != ValueType::U32) fail("general.alignment must be u32");
            const std::uint32_t a = v.scalar.u32;
            if (a == 0 || (a & (a - 1)) != 0) fail("general.alignment must be a positive power of two");
            f.alignment_ = a;
        }
        f.meta_index_.emplace(key, f.metadata_.size());
        f.metadata_.emplace_back(std::move(key), std::move(v));
    }

    struct Pending {
        std::string name;
        std::vector<std::int64_t> shape;
        std::uint32_t type;
        std::uint64_t offset;
    };
    std::vector<Pending> pend;
    pend.reserve(static_cast<std::size_t>(n_tensors));
    for (std::uint64_t i = 0; i < n_tensors; ++i) {
        Pending p;
        p.name = c.str();
        const std::uint32_t nd = c.get<std::uint32_t>();
        if (nd == 0 || nd > 8) fail("invalid tensor n_dims");
        p.shape.resize(nd);
        for (std::uint32_t d = 0; d < nd; ++d) p.shape[d] = static_cast<std::int64_t>(c.get<std::uint64_t>());
        p.type = c.get<std::uint32_t>();
        p.offset = c.get<std::uint64_t>();
        pend.push_back(std::move(p));
    }

    const std::size_t a = f.alignment_;
    const std::size_t blob = (c.pos + (a - 1)) & ~(a - 1);
    if (blob > f.size_ || blob < c.pos) fail("data blob start past end of file");

    f.tensors_.reserve(pend.size());
    for (Pending& p : pend) {
        TensorInfo info;
        info.name = std::move(p.name);
        info.shape = std::move(p.shape);
        info.ggml_type = p.type;
        std::int64_t numel = 1;
        for (std::int64_t d : info.shape) {
            if (d <= 0) fail("tensor '" + info.name + "' has non-positive dim");
            if (numel > INT64_MAX / d) fail("tensor numel overflows int64");
            numel *= d;
        }
        info.numel = numel;
        const TypeRow tr = type_row(p.type);
        info.dtype = tr.dtype;
        info.dtype_supported = tr.supported;
        std::size_t nbytes = 0;
        if (tr.supported) {
            if (tr.block > 1 && numel % tr.block != 0) fail("tensor '" + info.name + "' numel not multiple of block size");
            nbytes = static_cast<std::size_t>(numel / tr.block) * static_cast<std::size_t>(tr.bytes);
        }
        info.nbytes = nbytes;
        // bound the offset before adding it, and the size against what is left: a sum
        // that wraps would alias the tensor onto other bytes of the mapping
        if (p.offset > f.size_ || static_cast<std::size_t>(p.offset) > f.size_ - blob)
            fail("tensor '" + info.name + "' data out of bounds");
        const std::size_t abs = blob + static_cast<std::size_t>(p.offset);
        if (nbytes > f.size_ - abs) fail("tensor '" + info.name + "' data out of bounds");
        info.data = static_cast<const std::uint8_t*>(m) + abs;
        f.tensor_index_.emplace(info.name, f.tensors_.size());
        f.tensors_.push_back(std::move(info));
    }
    return f;
}

const TensorInfo* File::find_tensor(std::string_view name) const {
    auto it = tensor_index_.find(std::string(name));
    return it == tensor_index_.end() ? nullptr : &tensors_[it->second];
}
const TensorInfo& File::get_tensor(std::string_view name) const {
    const TensorInfo* t = find_tensor(name);
    if (!t) fail("no tensor named '" + std::string(name) + "'");
    return *t;
}
const Value* File::find_meta(std::string_view key) const {
    auto it = meta_index_.find(std::string(key));
    return it == meta_index_.end() ? nullptr : &metadata_[it->second].second;
}
const Value& File::get_meta(std::string_view key) const {
    const Value* v = find_meta(key);
    if (!v) fail("no metadata key '" + std::string(key) + "'");
    return *v;
}

// ---- shape / upload --------------------------------------------------------------------

std::pair<int, int> shape_to_2d(const std::vector<std::int64_t>& shape) {
    if (shape.empty()) fail("shape_to_2d: empty shape");
    for (std::int64_t d : shape) {
        if (d <= 0) fail("shape_to_2d: non-positive dimension");
        if (d > 0x7FFFFFFF) fail("shape_to_2d: dimension exceeds int range");
    }
    if (shape.size() == 1) return {static_cast<int>(shape[0]), 1};
    std::int64_t rows = 1;
    for (std::size_t i = 1; i < shape.size(); ++i) {
        if (rows > std::int64_t{0x7FFFFFFF} / shape[i]) fail("shape_to_2d: row product overflows int");
        rows *= shape[i];
    }
    return {static_cast<int>(rows), static_cast<int>(shape[0])};
}

namespace {

// Host bytes -> device through two pinned buffers: while one buffer is on its way to the
// device the next piece of the mapping is read (page-faulted) into the other one, by four threads (one
// thread copies at ~7 GB/s, a quarter of what the link takes). The buffers are allocated once per
// process (page-locking 2 x 32 MiB costs milliseconds) and uploads take turns on them.
struct PinnedPair {
    void* buf[2] = {nullptr, nullptr};
    cudaEvent_t ev[2] = {nullptr, nullptr};
    std::mutex mu;
    ~PinnedPair() {
        for (int i = 0; i < 2; ++i) {
            if (buf[i]) cudaFreeHost(buf[i]);
            if (ev[i]) cudaEventDestroy(ev[i]);
        }
    }
};
constexpr std::size_t kPiece = 32u << 20;
constexpr int kMaxCopyThreads = 16;
// Threads that fill a staging buffer: BROTENSOR_B200_UPLOAD_THREADS (1..16) or four. Measured on a 16-core host,
// 132 MB from the page cache: 4 threads 25.0-25.2 GB/s, 8: 25.9-27.8, 12: 27.6, 16: 25.9 - the copy out of the
// mapping, not the thread count, is what is left.
int copy_threads() {
    static const int n = [] {
        const char* e = std::getenv("BROTENSOR_B200_UPLOAD_THREADS");
        const int v = e ? std::atoi(e) : 0;
        return v >= 1 && v <= kMaxCopyThreads ? v : 4;
    }();
    return n;
}

void parallel_copy(void* dst, const std::uint8_t* src, std::size_t n) {
    const int kCopyThreads = copy_threads();
    if (n < (4u << 20) || kCopyThreads == 1) {
        std::memcpy(dst, src, n);
        return;
    }
    const std::size_t part = ((n / kCopyThreads) + 4095) & ~std::size_t(4095);
    std::thread th[kMaxCopyThreads - 1];
    for (int t = 1; t < kCopyThreads; ++t) {
        const std::size_t o = part * t;
        th[t - 1] = std::thread([=] {
            if (o < n) std::memcpy(static_cast<std::uint8_t*>(dst) + o, src + o, (n - o) < part ? (n - o) : part);
        });
    }
    std::memcpy(dst, src, n < part ? n : part);
    for (int t = 1; t < kCopyThreads; ++t) th[t - 1].join();
}

void staged_upload(void* dst, const std::uint8_t* src, std::size_t n, int dev) {
    static PinnedPair pp;
    std::lock_guard<std::mutex> lock(pp.mu);
    int prev = 0;
    cudaGetDevice(&prev);
    auto check = [&](cudaError_t e, const char* what) {
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            cudaSetDevice(prev);
            fail(std::string("upload: ") + what + ": " + cudaGetErrorString(e));
        }
    };
    check(cudaSetDevice(dev), "cudaSetDevice");
    cudaStream_t st = static_cast<cudaStream_t>(cuda_current_stream(dev));
    for (int i = 0; i < 2; ++i) {
        if (!pp.buf[i]) check(cudaMallocHost(&pp.buf[i], kPiece), "cudaMallocHost");
        if (!pp.ev[i]) check(cudaEventCreateWithFlags(&pp.ev[i], cudaEventDisableTiming), "cudaEventCreate");
    }
    std::size_t off = 0;
    for (int i = 0; off < n; ++i) {
        const int b = i & 1;
        const std::size_t len = (n - off) < kPiece ? (n - off) : kPiece;
        if (i >= 2) check(cudaEventSynchronize(pp.ev[b]), "cudaEventSynchronize");  // buffer b is free again
        parallel_copy(pp.buf[b], src + off, len);
        check(cudaMemcpyAsync(static_cast<std::uint8_t*>(dst) + off, pp.buf[b], len, cudaMemcpyHostToDevice, st), "cudaMemcpyAsync");
        check(cudaEventRecord(pp.ev[b], st), "cudaEventRecord");
        off += len;
    }
    check(cudaStreamSynchronize(st), "cudaStreamSynchronize");
    cudaSetDevice(prev);
}

void check_upload(const TensorInfo& info, int rows, int cols) {
    if (!info.dtype_supported)
        fail("upload_raw: tensor '" + info.name + "' has unsupported ggml_type " + std::to_string(info.ggml_type));
    if (rows <= 0 || cols <= 0) fail("upload_raw: rows/cols must be positive");
    const std::int64_t prod = static_cast<std::int64_t>(rows) * static_cast<std::int64_t>(cols);
    if (prod != info.numel)
        fail("upload_raw: rows*cols (" + std::to_string(prod) + ") != info.numel (" + std::to_string(info.numel) + ")");
    if (dtype_is_quant(info.dtype) && cols % dtype_block_size(info.dtype) != 0)
        fail("upload_raw: cols not a multiple of block size for quant dtype");
}

}  // namespace

void upload_rows(const TensorInfo& info, int rows, int cols, int row_begin, int row_end, Device target, Tensor& dst) {
    check_upload(info, rows, cols);
    if (row_begin < 0 || row_end < row_begin || row_end > rows) fail("upload_rows: row range out of bounds");
    const int n = row_end - row_begin;
    const std::size_t row_bytes = dtype_storage_bytes(info.dtype, cols);
    const std::uint8_t* src = info.data + static_cast<std::size_t>(row_begin) * row_bytes;
    const std::size_t nbytes = static_cast<std::size_t>(n) * row_bytes;
    if (target.is_cpu()) {
        dst = Tensor::from_raw_bytes_on(target, src, n, cols, info.dtype, nbytes);
        return;
    }
    dst = Tensor::empty_on(target, n, cols, info.dtype);
    if (nbytes) staged_upload(dst.data, src, nbytes, target.index);
}

void upload_rows_repacked(const TensorInfo& info, int rows, int cols, int row_begin, int row_end, Device target, Tensor& dst) {
    upload_rows(info, rows, cols, row_begin, row_end, target, dst);
    if (target.is_cuda() && dtype_is_quant(dst.dtype)) (void)repack_weights(dst);
}

void upload_raw(const TensorInfo& info, int rows, int cols, Tensor& dst) {
    upload_rows(info, rows, cols, 0, rows, default_device(), dst);
}

}  // namespace brotensor_b200::gguf

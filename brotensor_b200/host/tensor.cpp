// Tensor / Dtype / Device: storage through the backend allocator table, capacity-
// preserving resize, host <-> device copies. Behaviour follows brotensor's
// src/tensor.cpp (dtype sizing :50-133, from_raw_bytes_on :449-463, resize :543-571).
#include "brotensor_b200/tensor.h"

#include <cstring>
#include <stdexcept>
#include <utility>

#include "brotensor_b200/detail/dispatch.h"
#include "brotensor_b200/repack.h"
#include "brotensor_b200/runtime.h"

namespace brotensor_b200 {

const Device Device::CPU = Device(DeviceType::CPU, 0);
const Device Device::CUDA = Device(DeviceType::CUDA, 0);

namespace {
struct DtInfo { int size, block, block_bytes; };
DtInfo dt_info(Dtype d) {
    switch (d) {
        case Dtype::FP32: return {4, 1, 4};
        case Dtype::FP16: return {2, 1, 2};
        case Dtype::INT8: return {1, 1, 1};
        case Dtype::INT32: return {4, 1, 4};
        case Dtype::BF16: return {2, 1, 2};
        case Dtype::F64: return {8, 1, 8};
        case Dtype::Q4_0: return {0, 32, 18};
        case Dtype::Q4_1: return {0, 32, 20};
        case Dtype::Q5_0: return {0, 32, 22};
        case Dtype::Q5_1: return {0, 32, 24};
        case Dtype::Q8_0: return {0, 32, 34};
        case Dtype::Q8_1: return {0, 32, 36};
        case Dtype::Q2_K: return {0, 256, 82};
        case Dtype::Q3_K: return {0, 256, 110};
        case Dtype::Q4_K: return {0, 256, 144};
        case Dtype::Q5_K: return {0, 256, 176};
        case Dtype::Q6_K: return {0, 256, 210};
        case Dtype::Q8_K: return {0, 256, 292};
    }
    throw std::runtime_error("brotensor: unknown dtype");
}
[[noreturn]] void fail(const std::string& m) { throw std::runtime_error("brotensor: " + m); }
}  // namespace

int dtype_size_bytes(Dtype d) { return dt_info(d).size; }
int dtype_block_size(Dtype d) { return dt_info(d).block; }
int dtype_block_bytes(Dtype d) { return dt_info(d).block_bytes; }
bool dtype_is_quant(Dtype d) { return dt_info(d).size == 0; }
std::size_t dtype_storage_bytes(Dtype d, std::int64_t numel) {
    const DtInfo i = dt_info(d);
    if (numel < 0) fail("dtype_storage_bytes: negative element count");
    if (numel % i.block != 0) fail("dtype_storage_bytes: element count is not a multiple of the block size");
    return static_cast<std::size_t>(numel / i.block) * static_cast<std::size_t>(i.block_bytes);
}

const char* device_name(Device d) {
    switch (d.type) {
        case DeviceType::CPU: return "CPU";
        case DeviceType::CUDA: return "CUDA";
        case DeviceType::Metal: return "Metal";
    }
    return "?";
}
std::string to_string(Device d) {
    std::string s = device_name(d);
    if (d.type != DeviceType::CPU) s += ":" + std::to_string(d.index);
    return s;
}

// ---- lifecycle ---------------------------------------------------------------------

void Tensor::release_() {
    if (owns_ && data) {
        detail::forget_repacked(data);  // a later allocation at this address starts in the GGUF layout
        detail::alloc_for(device).free(data, device.index);
    }
    data = nullptr;
    owns_ = false;
    cap_bytes_ = 0;
}
Tensor::~Tensor() { release_(); }

Tensor::Tensor(Tensor&& o) noexcept
    : data(o.data), rows(o.rows), cols(o.cols), dtype(o.dtype), device(o.device), owns_(o.owns_), cap_bytes_(o.cap_bytes_) {
    o.data = nullptr;
    o.rows = o.cols = 0;
    o.owns_ = false;
    o.cap_bytes_ = 0;
}
Tensor& Tensor::operator=(Tensor&& o) noexcept {
    if (this != &o) {
        release_();
        data = o.data; rows = o.rows; cols = o.cols; dtype = o.dtype; device = o.device;
        owns_ = o.owns_; cap_bytes_ = o.cap_bytes_;
        o.data = nullptr;
        o.rows = o.cols = 0;
        o.owns_ = false;
        o.cap_bytes_ = 0;
    }
    return *this;
}
Tensor::Tensor(const Tensor& o) { *this = o.clone(); }
Tensor& Tensor::operator=(const Tensor& o) {
    if (this != &o) *this = o.clone();
    return *this;
}

std::size_t Tensor::bytes() const {
    return dtype_storage_bytes(dtype, static_cast<std::int64_t>(rows) * static_cast<std::int64_t>(cols));
}

Tensor Tensor::empty_on(Device dev, int r, int c, Dtype dt) {
    if (r < 0 || c < 0) fail("Tensor: negative dimension");
    Tensor t;
    t.rows = r; t.cols = c; t.dtype = dt; t.device = dev;
    const std::size_t n = t.bytes();
    if (n) {
        t.data = detail::alloc_for(dev).alloc(n, dev.index);
        t.owns_ = true;
        t.cap_bytes_ = n;
    }
    return t;
}
Tensor Tensor::zeros_on(Device dev, int r, int c, Dtype dt) {
    Tensor t = empty_on(dev, r, c, dt);
    t.zero();
    return t;
}
Tensor Tensor::zeros(int r, int c, Dtype dt) { return zeros_on(default_device(), r, c, dt); }
Tensor Tensor::empty(int r, int c, Dtype dt) { return empty_on(default_device(), r, c, dt); }

Tensor Tensor::from_raw_bytes_on(Device dev, const void* src, int r, int c, Dtype dt, std::size_t nbytes) {
    Tensor t = empty_on(dev, r, c, dt);
    if (nbytes != t.bytes()) fail("from_raw_bytes_on: nbytes does not match the tensor's storage size");
    if (nbytes) {
        if (!src) fail("from_raw_bytes_on: null source");
        if (dev.is_cpu()) std::memcpy(t.data, src, nbytes);
        else detail::alloc_for(dev).memcpy_h2d(t.data, src, nbytes, dev.index);
    }
    return t;
}
Tensor Tensor::from_host_on(Device dev, const float* src, int r, int c) {
    return from_raw_bytes_on(dev, src, r, c, Dtype::FP32, static_cast<std::size_t>(r) * c * 4);
}
Tensor Tensor::from_host_fp16_on(Device dev, const std::uint16_t* src, int r, int c) {
    return from_raw_bytes_on(dev, src, r, c, Dtype::FP16, static_cast<std::size_t>(r) * c * 2);
}
Tensor Tensor::from_host_bf16_on(Device dev, const std::uint16_t* src, int r, int c) {
    return from_raw_bytes_on(dev, src, r, c, Dtype::BF16, static_cast<std::size_t>(r) * c * 2);
}
Tensor Tensor::view(Device dev, void* p, int r, int c, Dtype dt) {
    Tensor t;
    t.data = p; t.rows = r; t.cols = c; t.dtype = dt; t.device = dev;
    return t;  // owns_ stays false
}

Tensor Tensor::clone() const { return to(device); }

namespace {
// A weight regrouped on the device (repack_weights) is a byte permutation of the GGUF block layout that
// only the device kernels read: host code handed those bytes would decode garbage without any error.
void refuse_regrouped_to_host(const Tensor& t, const char* what) {
    if (!t.device.is_cpu() && dtype_is_quant(t.dtype) && t.data && detail::repacked_ptr(t.data))
        fail(std::string(what) + ": the weight is in the regrouped device layout; call unpack_weights() first");
}
}  // namespace

Tensor Tensor::to(Device target) const {
    if (target.is_cpu()) refuse_regrouped_to_host(*this, "Tensor::to");
    Tensor t = empty_on(target, rows, cols, dtype);
    const std::size_t n = bytes();
    if (!n || !data) return t;
    if (device.is_cpu() && target.is_cpu()) std::memcpy(t.data, data, n);
    else if (device.is_cpu()) detail::alloc_for(target).memcpy_h2d(t.data, data, n, target.index);
    else if (target.is_cpu()) detail::alloc_for(device).memcpy_d2h(t.data, data, n, device.index);
    else if (device == target) detail::alloc_for(device).memcpy_d2d(t.data, data, n, device.index);
    else detail::alloc_for(device).memcpy_peer(t.data, target.index, data, device.index, n);
    // a byte copy of a whole regrouped weight is a regrouped weight
    if (dtype_is_quant(dtype) && detail::repacked_ptr(data)) detail::mark_repacked(t.data, n);
    return t;
}

void Tensor::zero() {
    const std::size_t n = bytes();
    if (n && data) detail::alloc_for(device).memset_zero(data, n, device.index);
}

void Tensor::resize(int r, int c, Dtype dt) {
    if (r < 0 || c < 0) fail("Tensor::resize: negative dimension");
    if (data && !owns_) fail("Tensor::resize: cannot resize a non-owning view");
    const std::size_t need = dtype_storage_bytes(dt, static_cast<std::int64_t>(r) * c);
    if (need > cap_bytes_) {
        release_();
        if (need) {
            data = detail::alloc_for(device).alloc(need, device.index);
            owns_ = true;
            cap_bytes_ = need;
        }
    }
    rows = r; cols = c; dtype = dt;
}

// ---- host round trips --------------------------------------------------------------

void Tensor::copy_raw_to_host(void* dst) const {
    const std::size_t n = bytes();
    if (!n) return;
    if (!data) fail("copy_to_host: tensor has no storage");
    refuse_regrouped_to_host(*this, "copy_to_host");
    if (device.is_cpu()) std::memcpy(dst, data, n);
    else detail::alloc_for(device).memcpy_d2h(dst, data, n, device.index);
}
// Stream-ordered forms for page-locked host memory (an extension over brotensor's Tensor,
// whose host round trips are blocking): enqueue on the calling thread's current stream and
// return; the data is valid after sync(device).
void Tensor::copy_raw_from_host_async(const void* src) {
    const std::size_t n = bytes();
    if (!n) return;
    if (!data) fail("copy_from_host_async: tensor has no storage");
    if (!src) fail("copy_from_host_async: null source");
    if (device.is_cpu()) std::memcpy(data, src, n);
    else detail::alloc_for(device).memcpy_h2d_async(data, src, n, device.index);
}
void Tensor::copy_raw_to_host_async(void* dst) const {
    const std::size_t n = bytes();
    if (!n) return;
    if (!data) fail("copy_to_host_async: tensor has no storage");
    refuse_regrouped_to_host(*this, "copy_to_host_async");
    if (device.is_cpu()) std::memcpy(dst, data, n);
    else detail::alloc_for(device).memcpy_d2h_async(dst, data, n, device.index);
}
void Tensor::copy_to_host(float* dst) const {
    if (dtype != Dtype::FP32) fail("copy_to_host: tensor is not FP32");
    copy_raw_to_host(dst);
}
void Tensor::copy_to_host_fp16(std::uint16_t* dst) const {
    if (dtype != Dtype::FP16) fail("copy_to_host_fp16: tensor is not FP16");
    copy_raw_to_host(dst);
}
void Tensor::copy_to_host_bf16(std::uint16_t* dst) const {
    if (dtype != Dtype::BF16) fail("copy_to_host_bf16: tensor is not BF16");
    copy_raw_to_host(dst);
}
std::vector<float> Tensor::to_host_vector() const {
    std::vector<float> v(static_cast<std::size_t>(size()));
    copy_to_host(v.data());
    return v;
}
std::vector<std::uint16_t> Tensor::to_host_vector_fp16() const {
    std::vector<std::uint16_t> v(static_cast<std::size_t>(size()));
    copy_to_host_fp16(v.data());
    return v;
}
std::vector<std::uint16_t> Tensor::to_host_vector_bf16() const {
    std::vector<std::uint16_t> v(static_cast<std::size_t>(size()));
    copy_to_host_bf16(v.data());
    return v;
}

// ---- scalar conversions (IEEE round to nearest even) -------------------------------

std::uint16_t fp32_to_fp16_bits(float v) {
    std::uint32_t x;
    std::memcpy(&x, &v, 4);
    const std::uint32_t sign = (x >> 16) & 0x8000u;
    const std::uint32_t e8 = (x >> 23) & 0xFFu;
    std::uint32_t man = x & 0x7FFFFFu;
    if (e8 == 0xFF) return static_cast<std::uint16_t>(sign | 0x7C00u | (man ? 0x0200u : 0u));
    const int e = static_cast<int>(e8) - 112;
    if (e >= 0x1F) return static_cast<std::uint16_t>(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return static_cast<std::uint16_t>(sign);
        man |= 0x800000u;
        const int shift = 14 - e;
        const std::uint32_t half = 1u << (shift - 1), rem = man & ((1u << shift) - 1u);
        std::uint32_t r = man >> shift;
        if (rem > half || (rem == half && (r & 1u))) ++r;
        return static_cast<std::uint16_t>(sign | r);
    }
    std::uint32_t out = (static_cast<std::uint32_t>(e) << 10) | (man >> 13);
    const std::uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (out & 1u))) ++out;
    if (out >= 0x7C00u) out = 0x7C00u;
    return static_cast<std::uint16_t>(sign | out);
}
float fp16_bits_to_fp32(std::uint16_t h) {
    const std::uint32_t sign = (static_cast<std::uint32_t>(h) & 0x8000u) << 16;
    std::uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, out;
    if (exp == 0) {
        if (man == 0) out = sign;
        else {
            int e = -1;
            do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
            out = sign | (static_cast<std::uint32_t>(112 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 0x1F) out = sign | 0x7F800000u | (man << 13);
    else out = sign | ((exp + 112u) << 23) | (man << 13);
    float f;
    std::memcpy(&f, &out, 4);
    return f;
}
std::uint16_t fp32_to_bf16_bits(float v) {
    std::uint32_t x;
    std::memcpy(&x, &v, 4);
    if ((x & 0x7F800000u) == 0x7F800000u && (x & 0x7FFFFFu)) return static_cast<std::uint16_t>((x >> 16) | 0x40u);
    x += 0x7FFFu + ((x >> 16) & 1u);
    return static_cast<std::uint16_t>(x >> 16);
}
float bf16_bits_to_fp32(std::uint16_t b) {
    const std::uint32_t x = static_cast<std::uint32_t>(b) << 16;
    float f;
    std::memcpy(&f, &x, 4);
    return f;
}

}  // namespace brotensor_b200

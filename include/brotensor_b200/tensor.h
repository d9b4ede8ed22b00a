// Tensor / Dtype / Device of the b200 host layer.
//
// Mirrors the part of brotensor's tensor surface that the GGUF quant-matmul path
// touches (include/brotensor/tensor.h:26-68 Dtype and block sizing, :76-109 Device,
// :130-291 Tensor): a row-major (rows, cols) buffer tagged with a Dtype and a
// Device, storage owned through the backend's allocator table, capacity-preserving
// resize so device pointers stay stable for CUDA-graph replay. Enum values are
// brotensor's, so a Dtype or Device crosses between the two libraries unchanged.
#pragma once

#include <cstddef>
#include <cstdint>
#include <functional>
#include <string>
#include <vector>

namespace brotensor_b200 {

enum class Dtype : int {
    FP32 = 0, FP16 = 1, INT8 = 2, INT32 = 3, BF16 = 4, F64 = 5,
    Q4_0 = 10, Q4_1 = 11, Q5_0 = 12, Q5_1 = 13, Q8_0 = 14, Q8_1 = 15,
    Q2_K = 20, Q3_K = 21, Q4_K = 22, Q5_K = 23, Q6_K = 24, Q8_K = 25,
};

int dtype_size_bytes(Dtype);   // bytes per scalar; 0 for block-quant carriers
int dtype_block_size(Dtype);   // elements per block (1 for scalars)
int dtype_block_bytes(Dtype);  // bytes per block (scalar size for scalars)
std::size_t dtype_storage_bytes(Dtype d, std::int64_t numel);  // throws if numel is not a block multiple
bool dtype_is_quant(Dtype);

enum class DeviceType : int { CPU = 0, CUDA = 1, Metal = 2 };

struct Device {
    DeviceType type = DeviceType::CPU;
    int index = 0;
    constexpr Device() = default;
    constexpr Device(DeviceType t, int idx = 0) : type(t), index(idx) {}
    static constexpr Device cpu() { return Device(DeviceType::CPU, 0); }
    static constexpr Device cuda(int idx = 0) { return Device(DeviceType::CUDA, idx); }
    static const Device CPU;
    static const Device CUDA;
    constexpr bool operator==(const Device& o) const { return type == o.type && index == o.index; }
    constexpr bool operator!=(const Device& o) const { return !(*this == o); }
    constexpr bool is_cpu() const { return type == DeviceType::CPU; }
    constexpr bool is_cuda() const { return type == DeviceType::CUDA; }
};

const char* device_name(Device);
std::string to_string(Device);

struct Tensor {
    void* data = nullptr;
    int rows = 0;  // rank-1: rows = N, cols = 1
    int cols = 0;
    Dtype dtype = Dtype::FP32;
    Device device = Device::CPU;

    Tensor() = default;
    ~Tensor();
    Tensor(const Tensor&);  // device-aware deep copy
    Tensor& operator=(const Tensor&);
    Tensor(Tensor&&) noexcept;
    Tensor& operator=(Tensor&&) noexcept;

    static Tensor zeros_on(Device, int r, int c, Dtype dt = Dtype::FP32);
    static Tensor empty_on(Device, int r, int c, Dtype dt = Dtype::FP32);
    static Tensor zeros(int r, int c, Dtype dt = Dtype::FP32);  // on the default device
    static Tensor empty(int r, int c, Dtype dt = Dtype::FP32);
    static Tensor from_host_on(Device, const float* src, int r, int c);
    static Tensor from_host_fp16_on(Device, const std::uint16_t* src, int r, int c);
    static Tensor from_host_bf16_on(Device, const std::uint16_t* src, int r, int c);
    // Any dtype, block-quant carriers included: nbytes must equal the tensor's bytes().
    static Tensor from_raw_bytes_on(Device, const void* src, int r, int c, Dtype dt, std::size_t nbytes);
    // Non-owning view; the destructor does not free `data`.
    static Tensor view(Device, void* data, int rows, int cols, Dtype = Dtype::FP32);

    Tensor to(Device target) const;
    Tensor clone() const;
    void zero();
    // Keeps the allocation whenever the new shape fits its capacity (pointer-stable);
    // contents are undefined afterwards. Throws on a negative dimension or on a view.
    void resize(int r, int c, Dtype dt = Dtype::FP32);

    int size() const { return rows * cols; }
    std::size_t bytes() const;
    bool empty() const { return data == nullptr || size() == 0; }
    bool owns_storage() const { return owns_; }  // false for Tensor::view results (not in brotensor)

    std::vector<float> to_host_vector() const;                // FP32 only
    std::vector<std::uint16_t> to_host_vector_fp16() const;   // FP16 only
    std::vector<std::uint16_t> to_host_vector_bf16() const;   // BF16 only
    void copy_to_host(float* dst) const;
    void copy_to_host_fp16(std::uint16_t* dst) const;
    void copy_to_host_bf16(std::uint16_t* dst) const;
    void copy_raw_to_host(void* dst) const;  // bytes() bytes, any dtype
    // Stream-ordered, non-blocking forms (not in brotensor): bytes() bytes between this tensor's
    // storage and page-locked host memory, on the calling thread's current stream.
    void copy_raw_from_host_async(const void* src);
    void copy_raw_to_host_async(void* dst) const;

private:
    bool owns_ = false;
    std::size_t cap_bytes_ = 0;
    void release_();
};

std::uint16_t fp32_to_fp16_bits(float v);
float fp16_bits_to_fp32(std::uint16_t bits);
std::uint16_t fp32_to_bf16_bits(float v);
float bf16_bits_to_fp32(std::uint16_t bits);

}  // namespace brotensor_b200

// mmap'd GGUF reader of the b200 host layer, plus the device upload path.
//
// Same reading contract as brotensor's loader (include/brotensor/gguf.h:27-115,
// src/gguf.cpp:317-445): versions 2 and 3, every metadata value type, up to 8
// dimensions, overflow-safe bounds checks, TensorInfo::data pointing into the
// mapping (valid while the File lives), shape_to_2d and upload_raw with the same
// errors ("gguf: <reason>"). New here: the upload stages the mapping through
// pinned double buffers with asynchronous copies, and upload_rows uploads a
// contiguous row range of a tensor (the per-GPU shard of a row-sharded weight).
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <string_view>
#include <unordered_map>
#include <utility>
#include <vector>

#include "tensor.h"

namespace brotensor_b200::gguf {

enum class ValueType : std::uint32_t {
    U8 = 0, I8 = 1, U16 = 2, I16 = 3, U32 = 4, I32 = 5, F32 = 6, Bool = 7, String = 8, Array = 9,
    U64 = 10, I64 = 11, F64 = 12,
};

struct Value {
    ValueType type = ValueType::U32;
    union Scalar {
        std::uint8_t u8; std::int8_t i8; std::uint16_t u16; std::int16_t i16;
        std::uint32_t u32; std::int32_t i32; std::uint64_t u64; std::int64_t i64;
        float f32; double f64; bool b;
    } scalar{};
    std::string str;
    ValueType array_elem_type = ValueType::U32;
    std::vector<Value> array;
};

struct TensorInfo {
    std::string name;
    std::vector<std::int64_t> shape;  // innermost first, as on disk
    std::uint32_t ggml_type = 0;
    Dtype dtype = Dtype::FP32;
    bool dtype_supported = true;
    const std::uint8_t* data = nullptr;
    std::size_t nbytes = 0;
    std::int64_t numel = 1;
};

class File {
public:
    File() = default;
    ~File();
    File(File&& other) noexcept;
    File& operator=(File&& other) noexcept;
    File(const File&) = delete;
    File& operator=(const File&) = delete;

    static File open(const std::string& path);

    const TensorInfo* find_tensor(std::string_view name) const;
    const TensorInfo& get_tensor(std::string_view name) const;
    const std::vector<TensorInfo>& tensors() const { return tensors_; }
    const Value* find_meta(std::string_view key) const;
    const Value& get_meta(std::string_view key) const;
    const std::vector<std::pair<std::string, Value>>& metadata() const { return metadata_; }
    std::uint32_t version() const { return version_; }
    std::uint32_t alignment() const { return alignment_; }
    std::size_t tensor_count() const { return tensors_.size(); }

private:
    void release_() noexcept;
    int fd_ = -1;
    void* base_ = nullptr;
    std::size_t size_ = 0;
    std::uint32_t version_ = 0;
    std::uint32_t alignment_ = 32;
    std::vector<std::pair<std::string, Value>> metadata_;
    std::unordered_map<std::string, std::size_t> meta_index_;
    std::vector<TensorInfo> tensors_;
    std::unordered_map<std::string, std::size_t> tensor_index_;
};

// (rows = product(shape[1..]), cols = shape[0]); 1-D -> (shape[0], 1).
std::pair<int, int> shape_to_2d(const std::vector<std::int64_t>& shape);

// Whole tensor to the default device as (rows, cols) of info.dtype; bytes unchanged.
void upload_raw(const TensorInfo& info, int rows, int cols, Tensor& dst);

// Rows [row_begin, row_end) of the (rows, cols) view of `info` to `target`: for a
// quantized tensor this is a contiguous byte range of the file, so a row-sharded
// weight needs no re-quantisation and each shard's content is bit-identical.
void upload_rows(const TensorInfo& info, int rows, int cols, int row_begin, int row_end, Device target, Tensor& dst);

// upload_rows followed by repack_weights (include/brotensor_b200/repack.h) on the target's current
// stream: the copy stays one contiguous byte range of the file, the regrouping happens on the
// device and is bit-identical in content. Opt-in: the ops take either layout.
void upload_rows_repacked(const TensorInfo& info, int rows, int cols, int row_begin, int row_end, Device target, Tensor& dst);

}  // namespace brotensor_b200::gguf

// Device-side repack of uploaded quantized weights (no counterpart in brotensor, which keeps the
// GGUF layout; its Q6_K kernels read it with 16-bit loads, src/cuda/detail/load_align.cuh:21-25).
//
// repack_weights() permutes a device-resident weight in place into the layout the B200 kernels
// read with aligned 16-byte loads; the tensor keeps its rows, cols, dtype and byte count, and the
// content is bit-identical (unpack_weights() restores the GGUF bytes exactly). Today one format
// has such a layout: Q6_K with cols % 2048 == 0, regrouped by field in runs of eight blocks
// (B200Q_FMT_Q6_K_R8 in include/b200q.h); for every other weight the call does nothing.
//
// Which layout a weight is in is recorded OUTSIDE the Tensor, by the address range of its storage,
// so brotensor's five public Tensor fields (include/brotensor/tensor.h:130-135) stay as they are and
// non-owning views of the whole weight or of a row range (a sharded LM head) are recognised too.
// The nine quant ops and the sharded head look the record up and pass the matching format code
// to the kernels; freeing the storage, or copying the tensor with clone() / to(), keeps it right.
#pragma once

#include <cstddef>

#include "brotensor_b200/tensor.h"

namespace brotensor_b200 {

// In place, on the calling thread's current stream of W's device. Returns true when W is in the
// regrouped layout afterwards (it was converted now or earlier), false when its format has none.
// Throws std::runtime_error("brotensor: repack_weights: <reason>") for a CPU tensor or a view.
bool repack_weights(Tensor& W);
// Back to the GGUF bytes; does nothing for a weight that is not regrouped.
void unpack_weights(Tensor& W);
// True when W.data lies inside storage recorded as regrouped.
bool is_repacked(const Tensor& W);

namespace detail {
void mark_repacked(const void* data, std::size_t nbytes);
void forget_repacked(const void* data);  // called when storage is freed
bool repacked_ptr(const void* data);
}  // namespace detail

}  // namespace brotensor_b200

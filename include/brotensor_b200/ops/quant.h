// The nine GGUF quant ops, with brotensor's signatures and argument meaning
// (include/brotensor/ops/quant.h:45-112).
//
//   dequant_*_to_fp16(W, W_fp16)                  W (out,in) quant -> (out,in), resized
//   linear_forward_*_fp16(W, bias, x, y)          y(out,1) = W x (+bias)
//   linear_forward_batched_*_fp16(W, bias, X, Y)  Y(B,out) = X(B,in) W^T (+bias)
//
// Superset of the reference contract: besides FP16, x / X may be FP32 or BF16 (bias
// has x's dtype). The output keeps its dtype when the caller pre-sized it as FP32,
// FP16 or BF16 with the right shape; otherwise it is resized to FP16 for FP16
// activations (the reference behaviour) and to FP32 for FP32 / BF16 activations.
// The dequant ops keep a pre-sized FP32 / BF16 destination likewise, else FP16.
// Errors are std::runtime_error("brotensor: <op>: <reason>") as in the reference.
#pragma once

#include <cstdint>

#include "../tensor.h"

namespace brotensor_b200 {

void dequant_q4k_to_fp16(const Tensor& W_q4k, Tensor& W_fp16);
void linear_forward_q4k_fp16(const Tensor& W_q4k, const Tensor* bias, const Tensor& x, Tensor& y);
void linear_forward_batched_q4k_fp16(const Tensor& W_q4k, const Tensor* bias, const Tensor& X_BD, Tensor& Y_BD);

void dequant_q8_0_to_fp16(const Tensor& W_q8, Tensor& W_fp16);
void linear_forward_q8_0_fp16(const Tensor& W_q8, const Tensor* bias, const Tensor& x, Tensor& y);
void linear_forward_batched_q8_0_fp16(const Tensor& W_q8, const Tensor* bias, const Tensor& X_BD, Tensor& Y_BD);

void dequant_q6k_to_fp16(const Tensor& W_q6k, Tensor& W_fp16);
void linear_forward_q6k_fp16(const Tensor& W_q6k, const Tensor* bias, const Tensor& x, Tensor& y);
void linear_forward_batched_q6k_fp16(const Tensor& W_q6k, const Tensor* bias, const Tensor& X_BD, Tensor& Y_BD);

// Extension: Q4_0 and Q5_K, which brotensor's GGUF loader hands out as opaque storage with no op behind
// them (src/gguf.cpp:111-130). Same three ops, shapes, dtypes and errors as for the formats above; the
// decode follows ggml's block definitions. They run on the plain-load GEMV (weights read once for up to
// eight activation rows), not on the streaming and tensor-core kernels.
void dequant_q4_0_to_fp16(const Tensor& W_q4_0, Tensor& W_fp16);
void linear_forward_q4_0_fp16(const Tensor& W_q4_0, const Tensor* bias, const Tensor& x, Tensor& y);
void linear_forward_batched_q4_0_fp16(const Tensor& W_q4_0, const Tensor* bias, const Tensor& X_BD, Tensor& Y_BD);
void dequant_q5k_to_fp16(const Tensor& W_q5k, Tensor& W_fp16);
void linear_forward_q5k_fp16(const Tensor& W_q5k, const Tensor* bias, const Tensor& x, Tensor& y);
void linear_forward_batched_q5k_fp16(const Tensor& W_q5k, const Tensor* bias, const Tensor& X_BD, Tensor& Y_BD);

// brotensor's embedding_lookup_forward (include/brotensor/ops/embedding.h:14-16) for a QUANTIZED table
// (Q4_K, Q6_K, Q8_0, Q4_0, Q5_K): out (B, D) = decode of the table rows d_idx[0..B), the same values as
// dequant_*_to_fp16 of those rows. d_idx: B int32 on the table's device. out is resized to (B, D) FP16
// unless it is pre-sized with that shape as FP32 / FP16 / BF16. brotensor throws for quantized tables
// ("quantized tables must be dequantized first", src/cuda/embedding.cu:150-154); a GGUF token_embd
// stored as Q4_K / Q6_K (and a tied LM head) needs no FP16 copy this way. An index outside [0, rows)
// yields a row of zeros (undefined in brotensor). FP32 / FP16 / BF16 tables are not this op's business
// and are refused.
void embedding_lookup_forward(const Tensor& table, const std::int32_t* d_idx, int B, Tensor& out);

// Extension (brotensor issues one launch per projection): n <= 4 weight matrices of ONE quant
// dtype (Q4_K, Q6_K or Q8_0) and one `in` against the same activation vector x (in, 1) in a
// single launch; y[s] = W[s] * x (+ bias[s]). A decode GEMV launch has a fixed cost of a few
// microseconds, which q/k/v or gate/up of a transformer layer pay once this way. Shapes, dtypes
// and error behaviour per matrix are those of linear_forward_q4k_fp16; results are bit-identical
// to n separate calls. `bias` may be null or hold null entries.
void linear_forward_group_fp16(const Tensor* const* W, const Tensor* const* bias, int n, const Tensor& x, Tensor* const* y);

// Extension (brotensor: two linear_forward_q4k_fp16 calls, a concat and swiglu_forward,
// include/brotensor/ops/activation.h:130-133): y (out, 1) = silu(W_gate x) * (W_up x) in one launch,
// silu(v) = v / (1 + exp(-v)). W_gate and W_up: (out, in) of one quant dtype; x (in, 1). y keeps a
// pre-sized FP32 / FP16 / BF16 dtype, else FP16 for FP16 x and FP32 otherwise.
void linear_forward_swiglu_fp16(const Tensor& W_gate, const Tensor& W_up, const Tensor& x, Tensor& y);

// Extension (brotensor: rms_norm_forward, include/brotensor/ops/norm.h:136-140, then one GEMV per
// projection): y[s] = W[s] * (x * gamma * rsqrt(mean(x^2) + eps)) for n <= 4 matrices of one quant
// dtype in a single launch; gamma (in, 1) of x's dtype. No bias. y as in linear_forward_group_fp16.
void linear_forward_group_rmsnorm_fp16(const Tensor* const* W, int n, const Tensor& x, const Tensor& gamma, float eps,
                                       Tensor* const* y);

}  // namespace brotensor_b200

/*
 * b200q — C-ABI of the B200 (sm_100a) GGUF fused quant-matmul backend.
 *
 * This is the whole boundary between a host library and the CUDA kernels:
 * plain pointers, sizes and a stream handle, no C++ or framework types. The
 * C++ host layer in brotensor_b200/host (Tensor / Device dispatch with
 * brotensor's op signatures) and the Python harness both sit on top of it.
 *
 * Every entry point works on the CUDA device that is current on the calling
 * thread (brotensor's dispatcher selects it before calling the backend slot,
 * src/dispatch.cpp:73-81), enqueues on `stream` (a cudaStream_t; NULL is the
 * legacy default stream) and returns without synchronising. Pointers are
 * device pointers unless stated otherwise. No entry point allocates or frees
 * device memory.
 *
 * Return value: B200Q_OK or one of the B200Q_ERR_* codes; b200q_last_error()
 * gives the message of the calling thread's most recent failure. There is no
 * CPU fallback: without a usable CUDA device every compute call fails with
 * B200Q_ERR_CUDA.
 */
#ifndef B200Q_H_
#define B200Q_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes. */
#define B200Q_OK 0
#define B200Q_ERR_BAD_ARG 1      /* null pointer, negative size, unknown format or dtype */
#define B200Q_ERR_UNSUPPORTED 2  /* legal arguments outside what the kernels cover */
#define B200Q_ERR_CUDA 3         /* a CUDA runtime call or launch failed */
#define B200Q_ERR_TIMEOUT 4      /* a bounded device-side wait ran out (see b200q_device_status) */
#define B200Q_ERR_WORKSPACE 5    /* workspace missing, misaligned or too small */

/* Block formats; the values are brotensor's Dtype tags (include/brotensor/tensor.h:26-47). */
#define B200Q_FMT_Q8_0 14 /*  32 elements /  34 B: fp16 d, int8 qs[32]                       */
#define B200Q_FMT_Q4_K 22 /* 256 elements / 144 B: fp16 d, fp16 dmin, u8 scales[12], u8 qs[128] */
#define B200Q_FMT_Q6_K 24 /* 256 elements / 210 B: u8 ql[128], u8 qh[64], i8 scales[16], fp16 d */
/*
 * Two more GGUF formats that brotensor's loader carries as opaque storage with no op behind them
 * (src/gguf.cpp:111-130); layouts as ggml defines them. Decode, dequant, decode GEMV, GEMM (as passes
 * of the GEMV) and the row gather take them; the tensor-core prefill kernel and the sharded head do not.
 */
#define B200Q_FMT_Q4_0 10 /*  32 elements /  18 B: fp16 d, u8 qs[16]; w = d * (nibble - 8), element j < 16 the low nibble of qs[j], else the high nibble of qs[j - 16] */
#define B200Q_FMT_Q5_K 23 /* 256 elements / 176 B: fp16 d, fp16 dmin, u8 scales[12] (packed as in Q4_K), u8 qh[32], u8 qs[128]; w = d * sc * (nibble + 16 * bit) - dmin * m */
/*
 * Q6_K repacked on the device in runs of eight blocks (b200q_repack): the same 1680 bytes per run,
 * regrouped by field - ql[8][128] @0, qh[8][64] @1024, scales[8][16] @1536, fp16 d[8] @1664 - so that
 * every field starts on a 16-byte boundary (raw Q6_K blocks are only 2-byte aligned). Content is
 * bit-identical (a byte permutation inside each run; b200q_unpack inverts it); K must be a multiple
 * of 2048. Accepted wherever B200Q_FMT_Q6_K is, except that W must be 16-byte aligned.
 */
#define B200Q_FMT_Q6_K_R8 124

/* Activation / output element types; the values are brotensor's Dtype tags. */
#define B200Q_DT_F32 0
#define B200Q_DT_F16 1
#define B200Q_DT_BF16 4

/* Library facts (no device needed). */
int b200q_abi_version(void);
const char* b200q_status_str(int status);
const char* b200q_last_error(void);
int b200q_block_elems(int fmt);                          /* 0 for an unknown format */
int b200q_block_bytes(int fmt);                          /* 0 for an unknown format */
size_t b200q_packed_bytes(int fmt, int64_t rows, int K); /* 0 if K is not a multiple of the block */

/*
 * Device-side repack of uploaded GGUF rows into the layout the kernels read fastest, and its inverse.
 * b200q_repacked_fmt: the format code of the repacked form of `fmt` for rows of K elements - Q6_K ->
 * Q6_K_R8 when K is a multiple of 2048; Q4_K and Q8_0 (whose bulk-copy granules are 16-byte aligned
 * as stored) and every other case return `fmt` itself, i.e. nothing to do. b200q_repack / b200q_unpack
 * move rows x K from `src` to `dst` (same byte count, b200q_packed_bytes; `dst == src` is allowed: a
 * run is read completely before it is written), `fmt` being the RAW format in both calls; with
 * nothing to do they copy (or return at once in place). No counterpart in the reference, which keeps
 * the raw layout (its kernels read Q6_K with 16-bit loads, src/cuda/detail/load_align.cuh:21-25).
 */
int b200q_repacked_fmt(int fmt, int K);
int b200q_repack(int fmt, const void* src, void* dst, int64_t rows, int K, void* stream);
int b200q_unpack(int fmt, const void* src, void* dst, int64_t rows, int K, void* stream);

/*
 * Block decode. W: rows x K quantized, row-major [rows][K/elems][block bytes];
 * out: rows x K of out_dtype. The FP32 result is the exact decoded value and
 * the 16-bit results are its round-to-nearest-even, i.e. bit-identical to the
 * reference's host decode.
 * Replaces dequant_q4k_to_fp16 / dequant_q6k_to_fp16 / dequant_q8_0_to_fp16
 * (include/brotensor/ops/quant.h:45,73,100; src/cuda/q4k.cu:297-324,
 * q6k.cu:232-259, q8_0.cu:195-222). Rows beyond 65535 are handled.
 */
int b200q_dequant(int fmt, const void* W, void* out, int out_dtype, int64_t rows, int K, void* stream);

/*
 * Row gather with decode, for a quantized embedding table (a GGUF token_embd stored as Q4_K / Q6_K /
 * Q8_0 / Q5_K / Q4_0, or a tied LM head): out[b][:] = decode(table row idx[b]) for b < B, the same
 * exact FP32 decode and single rounding as b200q_dequant of those rows. table: rows x K quantized;
 * idx: B int32 on the device; out: B x K of out_dtype, 16-byte aligned. An index outside [0, rows)
 * gives a row of zeros (brotensor leaves that case undefined, include/brotensor/ops/embedding.h:37-39;
 * nothing is read out of bounds here). brotensor's embedding_lookup_forward refuses quantized tables
 * (src/cuda/embedding.cu:150-154: "quantized tables must be dequantized first"), which costs a full
 * FP16 copy of the table; this op reads B rows of packed bytes.
 */
int b200q_embedding_gather(int fmt, const void* table, const int32_t* idx, int B, int64_t rows, int K, void* out, int out_dtype,
                           void* stream);

/*
 * Decode GEMV for 1..8 activation rows:
 *   Y(M,N) = X(M,K) * decode(W(N,K))^T (+ bias(N)),   FP32 accumulation.
 * X is M x K of x_dtype (row-major, leading dimension K), bias is N elements
 * of x_dtype or NULL, Y is M x N of y_dtype (leading dimension N). The weight
 * is streamed from HBM once whatever M is.
 * Replaces linear_forward_q4k_fp16 / _q6k_ / _q8_0_ (quant.h:52,79,105;
 * src/cuda/q4k.cu:326-362, q6k.cu:261-297, q8_0.cu:224-259) and the small-B
 * branch of the batched forms (q4k.cu:413-418, which re-reads W per row).
 */
int b200q_gemv(int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype,
               int M, int N, int K, void* stream);

/*
 * Several weight matrices of one format and one K against the SAME activation
 * vector (M = 1) in one launch: y_s(N_s) = decode(W_s(N_s,K)) * x (+ bias_s),
 * s = 0..n-1, n <= 4. A decode GEMV launch has a fixed cost of a few
 * microseconds; q/k/v or gate/up of a transformer layer pay it once this way.
 * Results are bit-identical to n calls of b200q_gemv. `bias` may be NULL or
 * hold NULL entries. brotensor issues one launch per projection
 * (src/cuda/q4k.cu:326-362); there is no grouped form in its op table.
 */
int b200q_gemv_multi(int fmt, int n, const void* const* W, const int* N, void* const* Y, const void* const* bias,
                     const void* x, int x_dtype, int y_dtype, int K, void* stream);

/*
 * b200q_gemv_multi with brotensor's rms_norm_forward (include/brotensor/ops/norm.h:136-140,
 * src/cuda/rms_norm.cu:56-75) folded into the kernel's activation staging: the n <= 4 matrices are
 * multiplied by x[j] * gamma[j] * rsqrt(mean_j x[j]^2 + eps), computed in FP32 by every CTA from the K
 * values of x, so the normalised vector is never written and the normalisation costs no launch.
 * gamma: K elements of x's dtype, 16-byte aligned. n = 1 is allowed. Shapes outside the streaming
 * kernel return B200Q_ERR_UNSUPPORTED (no fallback: the unfused form is rms_norm + b200q_gemv_multi).
 */
int b200q_gemv_multi_rmsnorm(int fmt, int n, const void* const* W, const int* N, void* const* Y, const void* const* bias,
                             const void* x, int x_dtype, const void* gamma, float eps, int y_dtype, int K, void* stream);

/*
 * Gate and up projection of a gated FFN in one launch, M = 1: y[i] = silu(W_gate[i] . x) * (W_up[i] . x),
 * silu(v) = v / (1 + exp(-v)) (brotensor's swiglu_forward, src/cuda/swiglu.cu:27-46, applied to the two
 * GEMV results without writing them out). W_gate and W_up: N x K of the same format, 16-byte aligned;
 * y: N elements. No bias. brotensor runs two linear_forward_q4k_fp16 calls and swiglu_forward.
 * Shapes outside the streaming kernel return B200Q_ERR_UNSUPPORTED.
 */
int b200q_gemv_swiglu(int fmt, const void* W_gate, const void* W_up, const void* x, int x_dtype, void* y, int y_dtype,
                      int N, int K, void* stream);

/*
 * Row-sharded decode GEMV for one rank of a multi-GPU LM head (M = 1):
 * this rank owns rows [row_offset, row_offset + rows) of a matrix of total_rows
 * rows; W_shard is the byte range of those rows, x is replicated. There is no
 * separate collective and, on the exchange path, no fence, flag or counter:
 * every CTA of the kernel sends its finished rows to ALL ranks through peer
 * pointers (NVLink stores) as 8-byte words that carry the value and the call's
 * number, and then receives its slice of the whole vector by polling the words
 * the peers sent - at most one second - and writing the values into this rank's
 * result vector. When the kernel has completed, this rank holds the whole
 * result vector.
 *   peer_out[q]   rank q's exchange memory, 24 * total_rows bytes: TWO result
 *                 vectors of total_rows FP32, used alternately (after the n-th
 *                 call on this state the result is vector (n & 1); only rank q
 *                 itself reads and writes them), then 2 x total_rows 8-byte
 *                 transfer words that every rank writes. Zero-initialised device
 *                 memory mapped into this process (e.g. CUDA IPC).
 *   state         this rank's own four uint32 (CTA counter, calls of both forms,
 *                 calls of the candidate form, reserved), zero-initialised; its
 *                 second word is the call count n.
 * All ranks must make the same sequence of calls. A rank that never sends
 * makes the others report B200Q_ERR_TIMEOUT through b200q_device_status(): the
 * kernel gives up after the wait limit (one second, or the "wait_limit_us"
 * option), records status 105 and returns; nothing traps or hangs. After such
 * a timeout this rank's call counter has advanced without its peers', so the
 * exchange memory of ALL ranks (peer_out, peer_cand, state) must be zeroed or
 * created anew before the head is used again; plain b200q_gemv calls on the
 * device are unaffected.
 * brotensor has no sharded form; the closest is its P2P bring-up
 * (src/cuda/register.cu:90-103).
 *
 * b200q_gemv_shard_topk is the candidate form for greedy / top-k sampling
 * (k = 1 .. 8, fewer than 1048575 rows, at most 256 CTAs): no logits cross the
 * links. Each rank keeps its shard's logits in its OWN result vector only;
 * every CTA reduces its rows to k candidates and stores them - value, row and a
 * tag of the call count in one indivisible 8-byte word each - into every rank's
 * candidate table; CTA 0 of each rank polls its table until all words carry
 * this call's tag (the same wait limit and timeout status) and leaves the k
 * best of all ranks in top_val (k FP32, largest first) and top_idx (k int32
 * global rows) on this device. Equal values keep the lower row, as brotensor's
 * greedy sampling does (include/brotensor/ops/sampling.h:27-28); top_idx[0] is
 * what sample_logits returns at temperature 0 on the full logit vector.
 *   peer_cand[q]  rank q's candidate table, 262144 bytes, zero-initialised,
 *                 mapped like peer_out: 2 x 8 x 256 x 8 uint64 (parity of the
 *                 call, writing rank, CTA slot, candidate).
 * The two forms may be mixed on one set of exchange memory.
 */
int b200q_gemv_shard(int fmt, const void* W_shard, const void* x, int x_dtype, const void* bias_shard, int rows, int K,
                     int row_offset, int total_rows, int rank, int world, void* const* peer_out, void* state, void* stream);
int b200q_gemv_shard_topk(int fmt, const void* W_shard, const void* x, int x_dtype, const void* bias_shard, int rows, int K,
                          int row_offset, int total_rows, int rank, int world, void* const* peer_out,
                          void* const* peer_cand, void* state, int k, void* top_val, void* top_idx, void* stream);

/*
 * Prefill GEMM on the tensor cores, any M >= 1:
 *   Y(M,N) = X(M,K) * decode(W(N,K))^T (+ bias(N)),   FP16 operands, FP32 accumulation.
 * `ws` is caller-owned scratch of at least b200q_gemm_workspace_bytes() bytes,
 * 256-byte aligned (it holds the activations converted to the operand layout
 * and, for matrices of few rows, whose k range is split over several CTA
 * pairs, the FP32 partial sums: splits x min(M, 512) x N floats);
 * it may be NULL when that size is 0. Calls that share a workspace must be
 * ordered on one stream.
 * Replaces the tensor-core branch of linear_forward_batched_q4k_fp16 / _q6k_ /
 * _q8_0_ (quant.h:61,87,111; src/cuda/q4k_wmma.cu:56-332, q6k_wmma.cu:62-377,
 * q8_0_wmma.cu:54-309).
 */
size_t b200q_gemm_workspace_bytes(int fmt, int x_dtype, int M, int N, int K);
int b200q_gemm(int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype,
               int M, int N, int K, void* ws, size_t ws_bytes, void* stream);

/*
 * b200q_gemm without a workspace argument and without any allocation: the
 * activation operand image goes to a fixed array in the library's own device
 * memory (b200q_gemm_static_max_bytes() bytes per device, 8 MiB: 512 tokens
 * at K = 8192, 1024 at K = 4096). For callers that cannot allocate: inside a
 * stream capture, under a fixed-footprint promise, or behind a plugin slot
 * that carries no workspace pointer. Problems whose
 * b200q_gemm_workspace_bytes() exceeds the array fail with
 * B200Q_ERR_WORKSPACE and nothing is launched.
 * All calls on one device share the one array: calls on the same stream are
 * ordered and safe; calls on different streams (or threads) that can overlap
 * race on it and must be ordered by the caller. Nothing in the array has to
 * be cleared between calls: every byte the GEMM reads is rewritten first.
 * The first call on a device does one-time set-up (symbol address lookup,
 * kernel attributes), so make one call before beginning a stream capture.
 * No counterpart in brotensor, whose batched ops allocate per call.
 */
size_t b200q_gemm_static_max_bytes(void);
int b200q_gemm_static(int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype,
                      int M, int N, int K, void* stream);

/*
 * Routing used by the batched ops: M <= 8 goes to b200q_gemv, larger M to
 * b200q_gemm (brotensor routes B >= 4 to its WMMA kernel, q4k_wmma.cu:320-326).
 */
int b200q_linear(int fmt, const void* W, const void* X, int x_dtype, const void* bias, void* Y, int y_dtype,
                 int M, int N, int K, void* ws, size_t ws_bytes, void* stream);

/*
 * How many tensor-core GEMM launches were made for `fmt` on this thread's
 * device since the last call; reading resets the count. The three named
 * aliases are the hooks brotensor's parity tests link against
 * (src/cuda/q4k_wmma.cu:337-348, q6k_wmma.cu:381-392, q8_0_wmma.cu:313-324).
 */
unsigned long long b200q_tc_calls_consume(int fmt);
unsigned long long brotensor_q4k_wmma_calls_consume(void);
unsigned long long brotensor_q6k_wmma_calls_consume(void);
unsigned long long brotensor_q8_0_wmma_calls_consume(void);

/*
 * Device-side status word of the current device: 0, or a code left by a kernel
 * whose bounded wait ran out (the kernel stops waiting and returns; it never
 * traps). Synchronises the device; reading resets the word.
 */
int b200q_device_status(int* status_out);

/*
 * Tuning knobs for benchmarks and tests (process-wide, not thread-safe):
 *   "gemv_path"   0 = automatic, 1 = plain-load kernel, 2 = warp-MMA streaming kernel,
 *                 3 = integer-dot streaming kernel (a forced path fails on shapes it does not take)
 *   "gemv_stages" ring depth of the streaming kernels (2..8); "gemv_stage_kb" stage size target;
 *   "gemv_grid"   CTA count (0 = one per SM)
 *   "pdl"         1 = launch GEMV kernels with programmatic dependent launch
 *   "gemv_groups" pipelines per CTA of the integer-dot kernel (1 or 2); "gemv_tile_pairs" 2 = prefer
 *                 one pipeline with 32-row tiles; "gemv_split_full" (Q6_K only) -1 = automatic, 0 = one full
 *                 barrier per stage, 1 = one per consumer warp and stage
 *   "gemm_path"   0 = automatic (tcgen05 GEMM from 9 rows, except 9..16 rows of Q4_K / Q8_0 with K = 2048 / 4096 and
 *                 of Q6_K from 8192 weight rows, which run as two passes of the small-batch GEMV), 1 = passes of the
 *                 decode GEMV only, 2 = the tcgen05 GEMM or an error
 *   "gemm_pair"   0 = one-CTA tcgen05 kernel, otherwise the CTA-pair kernel (default)
 *   "gemm_split"  0 = never split K; 1 (default) = matrices whose row tiles occupy at most half of the SMs
 *                 (N <= 9472) have their k-blocks split over up to eight CTA pairs, partial sums added in a
 *                 fixed order by a second kernel (b200q_gemm_workspace_bytes() grows accordingly)
 *   "gemv_xr"     Q4_K / Q6_K, one activation row, K <= 4096: 1 = the activation-resident kernel where it is the
 *                 faster one (default), 2 = for every such call, 0 = never
 *   "gemv_i8"     Q8_0 / Q4_K, 2..8 activation rows, K = 2048 / 4096: 1 = the integer tensor-core kernel where it is
 *                 the faster one (default), 2 = for every such call, 0 = never
 *   "gemv_lean"   0 = never take the trimmed instantiation of the integer-dot kernel (FP32 in and out, no bias)
 *   "wait_limit_us" bound of the decode kernels' device-side waits (stage barriers, peer arrival) in
 *                 microseconds; 0 = one second. Tests shorten it to see a wait run out.
 * Returns B200Q_ERR_BAD_ARG for an unknown key.
 */
int b200q_set_option(const char* key, int value);
int b200q_get_option(const char* key, int* value_out);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H_ */

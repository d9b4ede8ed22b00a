// Glue around the reference functions exported by the three shim TUs: the
// seeded input stream the reference tests draw from, row-level quantize /
// decode, and a row-parallel matmul that decodes each weight row with the
// reference's block decoder and accumulates sequentially in FP32 the way the
// reference tests do (tests/test_q4k_parity.cpp:267-274). Also exposes the
// reference GGUF reader for cross-checking the product's own parser.
// TEST INFRASTRUCTURE ONLY.
#include <brotensor/gguf.h>
#include <brotensor/tensor.h>

#include <cstdint>
#include <cstring>
#include <random>
#include <string>
#include <thread>
#include <vector>

extern "C" {
void ref_q4k_quantize_block(const float*, unsigned char*);
void ref_q4k_dequant_block(const unsigned char*, float*);
void ref_q6k_quantize_block(const float*, unsigned char*);
void ref_q6k_dequant_block(const unsigned char*, float*);
void ref_q8_0_quantize_block(const float*, unsigned char*);
void ref_q8_0_dequant_block(const unsigned char*, float*);
}

namespace {
std::mt19937 g_rng;
struct Fmt { int elems, bytes; void (*q)(const float*, unsigned char*); void (*dq)(const unsigned char*, float*); };
bool fmt_of(int fmt, Fmt& f) {
    switch (fmt) {
        case 22: f = {256, 144, ref_q4k_quantize_block, ref_q4k_dequant_block}; return true;
        case 24: f = {256, 210, ref_q6k_quantize_block, ref_q6k_dequant_block}; return true;
        case 14: f = {32, 34, ref_q8_0_quantize_block, ref_q8_0_dequant_block}; return true;
        default: return false;
    }
}
}  // namespace

extern "C" {

// The reference tests use one std::mt19937 per file and draw weights, then
// activations, then bias from std::uniform_real_distribution<float>.
void ref_rng_seed(uint32_t seed) { g_rng.seed(seed); }
void ref_rng_uniform(float lo, float hi, int64_t n, float* out) {
    std::uniform_real_distribution<float> d(lo, hi);
    for (int64_t i = 0; i < n; ++i) out[i] = d(g_rng);
}

uint16_t ref_fp32_to_fp16_bits(float v) { return brotensor::fp32_to_fp16_bits(v); }
float ref_fp16_bits_to_fp32(uint16_t b) { return brotensor::fp16_bits_to_fp32(b); }
uint16_t ref_fp32_to_bf16_bits(float v) { return brotensor::fp32_to_bf16_bits(v); }
float ref_bf16_bits_to_fp32(uint16_t b) { return brotensor::bf16_bits_to_fp32(b); }

int ref_quantize_rows(int fmt, const float* Wf, int64_t rows, int K, unsigned char* out) {
    Fmt f;
    if (!fmt_of(fmt, f) || K % f.elems) return -1;
    const int bpr = K / f.elems;
    for (int64_t r = 0; r < rows; ++r)
        for (int b = 0; b < bpr; ++b)
            f.q(Wf + r * K + (int64_t)b * f.elems, out + (r * bpr + b) * f.bytes);
    return 0;
}

int ref_dequant_rows(int fmt, const unsigned char* W, int64_t rows, int K, float* out) {
    Fmt f;
    if (!fmt_of(fmt, f) || K % f.elems) return -1;
    const int bpr = K / f.elems;
    for (int64_t r = 0; r < rows; ++r)
        for (int b = 0; b < bpr; ++b)
            f.dq(W + (r * bpr + b) * f.bytes, out + r * K + (int64_t)b * f.elems);
    return 0;
}

// Y(M,N) = X(M,K) * decode(W(N,K))^T (+bias). Rows split over `threads`.
int ref_matmul(int fmt, const unsigned char* W, const float* X, const float* bias, float* Y,
               int M, int N, int K, int threads) {
    Fmt f;
    if (!fmt_of(fmt, f) || K % f.elems) return -1;
    const int bpr = K / f.elems;
    if (threads < 1) threads = 1;
    auto work = [&](int64_t r0, int64_t r1) {
        std::vector<float> row(K);
        for (int64_t r = r0; r < r1; ++r) {
            for (int b = 0; b < bpr; ++b) f.dq(W + (r * bpr + b) * f.bytes, row.data() + (int64_t)b * f.elems);
            for (int m = 0; m < M; ++m) {
                const float* x = X + (int64_t)m * K;
                float s = 0.0f;
                for (int k = 0; k < K; ++k) s += row[k] * x[k];
                Y[(int64_t)m * N + r] = bias ? s + bias[r] : s;
            }
        }
    };
    if (threads == 1) { work(0, N); return 0; }
    std::vector<std::thread> th;
    for (int t = 0; t < threads; ++t) th.emplace_back(work, (int64_t)N * t / threads, (int64_t)N * (t + 1) / threads);
    for (auto& t : th) t.join();
    return 0;
}

// Reference GGUF reader: opens `path`, returns the tensor count (or -1 and a
// message in err). Tensor i's fields are read back with ref_gguf_tensor.
static brotensor::gguf::File* g_file = nullptr;
int ref_gguf_open(const char* path, char* err, int errlen) {
    try {
        delete g_file;
        g_file = nullptr;
        g_file = new brotensor::gguf::File(brotensor::gguf::File::open(path));
        return (int)g_file->tensor_count();
    } catch (const std::exception& e) {
        if (err && errlen > 0) { std::strncpy(err, e.what(), errlen - 1); err[errlen - 1] = 0; }
        return -1;
    }
}
int ref_gguf_tensor(int i, char* name, int namelen, int64_t* shape8, int* ndims, uint32_t* ggml_type,
                    int* dtype, int* supported, uint64_t* nbytes, int64_t* numel, uint64_t* data_off_in_first_tensor) {
    if (!g_file || i < 0 || i >= (int)g_file->tensor_count()) return -1;
    const auto& t = g_file->tensors()[i];
    std::strncpy(name, t.name.c_str(), namelen - 1);
    name[namelen - 1] = 0;
    *ndims = (int)t.shape.size();
    for (int d = 0; d < *ndims && d < 8; ++d) shape8[d] = t.shape[d];
    *ggml_type = t.ggml_type;
    *dtype = (int)t.dtype;
    *supported = t.dtype_supported ? 1 : 0;
    *nbytes = t.nbytes;
    *numel = t.numel;
    *data_off_in_first_tensor = (uint64_t)(t.data - g_file->tensors()[0].data);
    return 0;
}
uint32_t ref_gguf_alignment() { return g_file ? g_file->alignment() : 0; }
uint32_t ref_gguf_version() { return g_file ? g_file->version() : 0; }
void ref_gguf_close() { delete g_file; g_file = nullptr; }
int ref_shape_to_2d(const int64_t* shape, int n, int* rows, int* cols, char* err, int errlen) {
    try {
        auto rc = brotensor::gguf::shape_to_2d(std::vector<int64_t>(shape, shape + n));
        *rows = rc.first; *cols = rc.second;
        return 0;
    } catch (const std::exception& e) {
        if (err && errlen > 0) { std::strncpy(err, e.what(), errlen - 1); err[errlen - 1] = 0; }
        return -1;
    }
}
}

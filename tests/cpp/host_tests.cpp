// Tests of the C++ host layer, in the style of brotensor's own test executables
// (a CHECK macro and a failure counter; tests/test_q4k_parity.cpp:36-37):
//   host_tests cpu   tensor / dispatch / GGUF reader behaviour, no GPU touched
//                    (cases after tests/test_tensor_errors.cpp:556-589, tests/test_gguf.cpp,
//                    tests/test_gguf_extra.cpp:233-290, 470-482, 598-608, 638-810)
//   host_tests gpu   the nine quant ops through Tensor / dispatch on CUDA, checked against
//                    the CPU oracle (cases after tests/test_q4k_parity.cpp A-G and
//                    tests/test_q8_0_parity.cpp H)
#include <cuda_runtime_api.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <functional>
#include <stdexcept>
#include <string>
#include <vector>

#include "b200q.h"
#include "brotensor_b200/detail/dispatch.h"
#include "brotensor_b200/gguf.h"
#include "brotensor_b200/ops/quant.h"
#include "brotensor_b200/repack.h"
#include "brotensor_b200/runtime.h"

namespace bt = brotensor_b200;
using bt::Device;
using bt::Dtype;
using bt::Tensor;

extern "C" {  // the CPU oracle (test infrastructure)
int oracle_dequant_f32(int fmt, const uint8_t* W, int64_t rows, int K, float* out);
int oracle_dequant_16(int fmt, const uint8_t* W, int64_t rows, int K, int kind, uint16_t* out);
int oracle_matmul(int fmt, const uint8_t* W, const float* X, const float* bias, float* Y, double* Y64, int M, int N,
                  int K, int threads);
}

static int g_failures = 0;
#define CHECK(c) do { if (!(c)) { std::printf("  FAIL %s:%d %s\n", __FILE__, __LINE__, #c); ++g_failures; } } while (0)

static bool throws_with(const std::function<void()>& f, const char* needle) {
    try {
        f();
    } catch (const std::runtime_error& e) {
        if (std::strstr(e.what(), needle)) return true;
        std::printf("  message was: %s\n", e.what());
        return false;
    }
    return false;
}

// ---------------------------------------------------------------- GGUF fixture writer
struct Gguf {
    std::vector<uint8_t> b;
    template <typename T> void put(T v) { const uint8_t* p = reinterpret_cast<const uint8_t*>(&v); b.insert(b.end(), p, p + sizeof(T)); }
    void str(const std::string& s) { put<uint64_t>(s.size()); b.insert(b.end(), s.begin(), s.end()); }
    void header(uint32_t version, uint64_t nt, uint64_t nm) { put<uint32_t>(0x46554747u); put(version); put(nt); put(nm); }
    void tensor(const std::string& name, std::vector<uint64_t> dims, uint32_t type, uint64_t off) {
        str(name); put<uint32_t>((uint32_t)dims.size());
        for (auto d : dims) put<uint64_t>(d);
        put(type); put(off);
    }
    void pad(size_t a) { while (b.size() % a) b.push_back(0); }
    std::string write(const char* tag) {
        std::string path = std::string("/tmp/b200_gguf_") + tag + ".gguf";
        std::ofstream(path, std::ios::binary).write(reinterpret_cast<const char*>(b.data()), (std::streamsize)b.size());
        return path;
    }
};

static void test_cpu_tensor_and_dispatch() {
    std::printf("test_cpu_tensor_and_dispatch\n");
    CHECK(bt::dtype_block_size(Dtype::Q4_K) == 256 && bt::dtype_block_bytes(Dtype::Q4_K) == 144);
    CHECK(bt::dtype_block_size(Dtype::Q6_K) == 256 && bt::dtype_block_bytes(Dtype::Q6_K) == 210);
    CHECK(bt::dtype_block_size(Dtype::Q8_0) == 32 && bt::dtype_block_bytes(Dtype::Q8_0) == 34);
    CHECK(bt::dtype_storage_bytes(Dtype::Q4_K, 4096LL * 4096) == 9437184u);
    CHECK(bt::dtype_size_bytes(Dtype::Q4_K) == 0 && bt::dtype_is_quant(Dtype::Q8_0) && !bt::dtype_is_quant(Dtype::BF16));
    CHECK(throws_with([] { bt::dtype_storage_bytes(Dtype::Q4_K, 100); }, "multiple of the block size"));

    Tensor t = Tensor::zeros_on(Device::CPU, 4, 256, Dtype::Q4_K);
    CHECK(t.bytes() == 4 * 144 && t.data != nullptr);
    void* p = t.data;
    t.resize(2, 256, Dtype::Q4_K);
    CHECK(t.data == p);  // shrinking keeps the allocation (pointer-stable)
    t.resize(4, 256, Dtype::Q4_K);
    CHECK(t.data == p);
    Tensor c = t;  // deep copy
    CHECK(c.data != t.data && c.bytes() == t.bytes());
    Tensor m = std::move(c);
    CHECK(c.data == nullptr && m.data != nullptr);
    std::vector<float> backing(4, 0.f);
    Tensor v = Tensor::view(Device::CPU, backing.data(), 2, 2);
    CHECK(throws_with([&] { v.resize(4, 4); }, "view"));
    CHECK(throws_with([&] { Tensor::empty_on(Device::CPU, -1, 2); }, "negative"));
    CHECK(throws_with([&] { Tensor::from_raw_bytes_on(Device::CPU, backing.data(), 2, 2, Dtype::FP32, 15); }, "nbytes"));

    // fp16 / bf16 conversions round to nearest even and round-trip every finite fp16
    for (uint32_t h = 0; h < 65536; ++h) {
        const float f = bt::fp16_bits_to_fp32((uint16_t)h);
        if (std::isnan(f)) continue;
        if (bt::fp32_to_fp16_bits(f) != h) { CHECK(false); break; }
    }
    CHECK(bt::fp32_to_fp16_bits(1.00048828125f) == 0x3C00);  // tie to even
    CHECK(bt::fp32_to_bf16_bits(1.0f) == 0x3F80 && bt::bf16_bits_to_fp32(0x3F80) == 1.0f);

    // dispatch: a CUDA-tagged non-owning view over host memory provokes the mismatch
    // without touching a GPU
    Tensor cpu_t = Tensor::zeros_on(Device::CPU, 2, 2);
    Tensor other = Tensor::view(Device::CUDA, backing.data(), 2, 2);
    CHECK(throws_with([&] { (void)&bt::detail::dispatch_with_opts(cpu_t, {&other}); }, "but the op resolved to CPU"));
    CHECK(throws_with([&] { (void)&bt::detail::dispatch_with_opts(cpu_t, {nullptr, &other}); }, "operand 2"));

    // the CPU backend has no quant ops (as in the reference): null slot -> "not implemented on CPU"
    Tensor w = Tensor::zeros_on(Device::CPU, 1, 256, Dtype::Q4_K), o = Tensor::zeros_on(Device::CPU, 1, 256, Dtype::FP16);
    CHECK(throws_with([&] { bt::dequant_q4k_to_fp16(w, o); }, "dequant_q4k_to_fp16: not implemented on CPU"));
    Tensor x = Tensor::zeros_on(Device::CPU, 256, 1, Dtype::FP16), y;
    CHECK(throws_with([&] { bt::linear_forward_q4k_fp16(w, nullptr, x, y); }, "linear_forward_q4k_fp16: not implemented on CPU"));
    CHECK(throws_with([&] { bt::linear_forward_batched_q6k_fp16(w, nullptr, x, y); }, "not implemented on CPU"));
}

static void test_cpu_gguf() {
    std::printf("test_cpu_gguf\n");
    // a valid v3 file: every metadata type, a nested array, four tensors incl. an unknown type
    Gguf g;
    g.header(3, 4, 6);
    g.str("general.alignment"); g.put<uint32_t>(4); g.put<uint32_t>(64);
    g.str("a.u8"); g.put<uint32_t>(0); g.put<uint8_t>(7);
    g.str("a.str"); g.put<uint32_t>(8); g.str("hello");
    g.str("a.f64"); g.put<uint32_t>(12); g.put<double>(2.5);
    g.str("a.bool"); g.put<uint32_t>(7); g.put<uint8_t>(1);
    g.str("a.arr"); g.put<uint32_t>(9); g.put<uint32_t>(9); g.put<uint64_t>(2);  // array of arrays
    for (int i = 0; i < 2; ++i) { g.put<uint32_t>(5); g.put<uint64_t>(3); for (int j = 0; j < 3; ++j) g.put<int32_t>(i * 3 + j); }
    g.tensor("w.q4k", {512, 4}, 12, 0);          // 4 rows x 2 blocks = 1152 B
    g.tensor("w.q6k", {256, 2, 3}, 14, 1152);    // 6 rows x 1 block = 1260 B
    g.tensor("w.q8_0", {64}, 8, 1152 + 1280);    // 1-D: 2 blocks = 68 B
    g.tensor("w.unknown", {8}, 99, 0);
    g.pad(64);
    const size_t blob = g.b.size();
    for (int i = 0; i < 1152 + 1280 + 68; ++i) g.b.push_back((uint8_t)(i * 7 + 3));
    const std::string path = g.write("ok");
    {
        bt::gguf::File f = bt::gguf::File::open(path);
        CHECK(f.version() == 3 && f.alignment() == 64 && f.tensor_count() == 4 && f.metadata().size() == 6);
        CHECK(f.get_meta("a.str").str == "hello" && f.get_meta("a.u8").scalar.u8 == 7 && f.get_meta("a.bool").scalar.b);
        CHECK(f.get_meta("a.arr").array.size() == 2 && f.get_meta("a.arr").array[1].array[2].scalar.i32 == 5);
        CHECK(f.find_meta("nope") == nullptr);
        CHECK(throws_with([&] { f.get_meta("nope"); }, "no metadata key"));
        const auto& q4 = f.get_tensor("w.q4k");
        CHECK(q4.dtype == Dtype::Q4_K && q4.nbytes == 1152 && q4.numel == 2048 && q4.dtype_supported);
        CHECK(q4.data[0] == 3 && q4.data[1] == 10);
        const auto& q6 = f.get_tensor("w.q6k");
        CHECK(q6.dtype == Dtype::Q6_K && q6.nbytes == 1260 && q6.data == q4.data + 1152);
        auto rc = bt::gguf::shape_to_2d(q6.shape);
        CHECK(rc.first == 6 && rc.second == 256);
        CHECK(bt::gguf::shape_to_2d(f.get_tensor("w.q8_0").shape) == std::make_pair(64, 1));
        const auto& un = f.get_tensor("w.unknown");
        CHECK(!un.dtype_supported && un.nbytes == 0);
        CHECK(throws_with([&] { f.get_tensor("missing"); }, "no tensor named"));
        // uploads (default device is the CPU here): bytes unchanged, row ranges are byte ranges
        Tensor w;
        bt::gguf::upload_raw(q4, 4, 512, w);
        CHECK(w.dtype == Dtype::Q4_K && w.rows == 4 && w.cols == 512 && !std::memcmp(w.data, q4.data, 1152));
        Tensor part;
        bt::gguf::upload_rows(q4, 4, 512, 1, 3, Device::CPU, part);
        CHECK(part.rows == 2 && !std::memcmp(part.data, q4.data + 288, 576));
        CHECK(throws_with([&] { bt::gguf::upload_raw(un, 8, 1, w); }, "unsupported ggml_type 99"));
        CHECK(throws_with([&] { bt::gguf::upload_raw(q4, 4, 500, w); }, "!= info.numel"));
        CHECK(throws_with([&] { bt::gguf::upload_raw(q4, 16, 128, w); }, "cols not a multiple of block size"));
        CHECK(throws_with([&] { bt::gguf::upload_raw(f.get_tensor("w.q8_0"), 64, 1, w); }, "cols not a multiple of block size"));
        CHECK(throws_with([&] { bt::gguf::upload_raw(q4, 0, 512, w); }, "must be positive"));
        CHECK(throws_with([&] { bt::gguf::upload_rows(q4, 4, 512, 2, 5, Device::CPU, w); }, "row range"));
        bt::gguf::File moved = std::move(f);
        CHECK(moved.tensor_count() == 4 && f.tensor_count() == 0);
    }
    (void)blob;
    CHECK(throws_with([] { bt::gguf::shape_to_2d({}); }, "empty shape"));
    CHECK(throws_with([] { bt::gguf::shape_to_2d({4, 0}); }, "non-positive"));
    CHECK(throws_with([] { bt::gguf::shape_to_2d({4, int64_t(1) << 40}); }, "exceeds int range"));
    CHECK(throws_with([] { bt::gguf::shape_to_2d({2, 70000, 70000}); }, "overflows int"));

    // malformed files
    auto bad = [&](const char* tag, const std::function<void(Gguf&)>& build, const char* needle) {
        Gguf m;
        build(m);
        const std::string p = m.write(tag);
        CHECK(throws_with([&] { bt::gguf::File::open(p); }, needle));
    };
    bad("magic", [](Gguf& m) { m.put<uint32_t>(0x12345678u); m.put<uint32_t>(3); m.put<uint64_t>(0); m.put<uint64_t>(0); }, "bad magic");
    bad("version", [](Gguf& m) { m.header(1, 0, 0); }, "unsupported GGUF version 1");
    bad("small", [](Gguf& m) { m.put<uint32_t>(0x46554747u); }, "file too small");
    bad("eof", [](Gguf& m) { m.header(3, 0, 1); m.str("k"); m.put<uint32_t>(8); m.put<uint64_t>(1000); m.put<uint32_t>(0); }, "unexpected EOF");
    bad("hugestr", [](Gguf& m) { m.header(3, 0, 1); m.put<uint64_t>(~0ull - 3); m.put<uint64_t>(0); m.put<uint64_t>(0); }, "unexpected EOF");
    bad("vtype", [](Gguf& m) { m.header(3, 0, 1); m.str("k"); m.put<uint32_t>(13); m.put<uint64_t>(0); }, "value type out of range");
    bad("bool", [](Gguf& m) { m.header(3, 0, 1); m.str("k"); m.put<uint32_t>(7); m.put<uint8_t>(2); m.put<uint64_t>(0); m.put<uint64_t>(0); }, "bool value");
    bad("align0", [](Gguf& m) { m.header(3, 0, 1); m.str("general.alignment"); m.put<uint32_t>(4); m.put<uint32_t>(24); m.put<uint64_t>(0); }, "power of two");
    bad("alignty", [](Gguf& m) { m.header(3, 0, 1); m.str("general.alignment"); m.put<uint32_t>(10); m.put<uint64_t>(32); m.put<uint64_t>(0); }, "must be u32");
    bad("ndims", [](Gguf& m) { m.header(3, 1, 0); m.str("t"); m.put<uint32_t>(9); m.put<uint64_t>(0); m.put<uint64_t>(0); }, "invalid tensor n_dims");
    bad("dim0", [](Gguf& m) { m.header(3, 1, 0); m.tensor("t", {0}, 0, 0); m.pad(32); }, "non-positive dim");
    bad("numelov", [](Gguf& m) { m.header(3, 1, 0); m.tensor("t", {1ull << 40, 1ull << 40}, 0, 0); m.pad(32); }, "overflows int64");
    bad("block", [](Gguf& m) { m.header(3, 1, 0); m.tensor("t", {100}, 12, 0); m.pad(32); }, "not multiple of block size");
    bad("oob", [](Gguf& m) { m.header(3, 1, 0); m.tensor("t", {256}, 12, 0); m.pad(32); for (int i = 0; i < 100; ++i) m.b.push_back(0); }, "data out of bounds");
    bad("offwrap", [](Gguf& m) { m.header(3, 1, 0); m.tensor("t", {256}, 12, ~0ull - 8); m.pad(32); for (int i = 0; i < 200; ++i) m.b.push_back(0); }, "data out of bounds");
    CHECK(throws_with([] { bt::gguf::File::open("/tmp/definitely_not_here.gguf"); }, "cannot open"));
}

// ---------------------------------------------------------------- GPU cases
struct FmtCase {
    const char* name;
    int fmt;
    Dtype dt;
    int block, bytes;
    void (*dequant)(const Tensor&, Tensor&);
    void (*gemv)(const Tensor&, const Tensor*, const Tensor&, Tensor&);
    void (*batched)(const Tensor&, const Tensor*, const Tensor&, Tensor&);
    unsigned long long (*tc_calls)();
};

static uint32_t g_lcg = 0x1234567u;
static uint32_t lcg() { g_lcg = g_lcg * 1664525u + 1013904223u; return g_lcg; }
static float frand(float lo, float hi) { return lo + (hi - lo) * (float(lcg() >> 8) / float(1u << 24)); }

// Random block bytes with the fp16 scale fields pinned to finite values
// (the construction of tests/test_quant_prefill_parity.cpp:67-88).
static std::vector<uint8_t> make_blocks(const FmtCase& c, int rows, int K) {
    const size_t nb = (size_t)rows * (K / c.block);
    std::vector<uint8_t> b(nb * c.bytes);
    for (auto& v : b) v = (uint8_t)(lcg() >> 24);
    for (size_t i = 0; i < nb; ++i) {
        uint8_t* p = &b[i * c.bytes];
        auto put = [&](int off, float f) { const uint16_t h = bt::fp32_to_fp16_bits(f); p[off] = h & 0xFF; p[off + 1] = h >> 8; };
        if (c.fmt == B200Q_FMT_Q4_K) { put(0, 0.02f * frand(0.5f, 1.5f)); put(2, 0.008f * frand(0.5f, 1.5f)); }
        else if (c.fmt == B200Q_FMT_Q8_0) put(0, 0.01f * frand(0.5f, 1.5f));
        else put(c.bytes - 2, 0.01f * frand(0.5f, 1.5f));
    }
    return b;
}

static double rel_l2(const std::vector<float>& got, const std::vector<float>& want) {
    double num = 0, den = 0;
    for (size_t i = 0; i < got.size(); ++i) { const double d = (double)got[i] - want[i]; num += d * d; den += (double)want[i] * want[i]; }
    return std::sqrt(num) / (den > 0 ? std::sqrt(den) : 1.0);
}

static void run_fmt(const FmtCase& c) {
    std::printf("test_gpu_%s\n", c.name);
    const Device dev = Device::CUDA;
    const int OUT = 64, IN = c.fmt == B200Q_FMT_Q8_0 ? 256 : 512;
    const std::vector<uint8_t> Wb = make_blocks(c, OUT, IN);
    Tensor W = Tensor::empty_on(dev, OUT, IN, c.dt);
    cudaMemcpy(W.data, Wb.data(), Wb.size(), cudaMemcpyHostToDevice);  // tests write raw blocks into W.data

    // A: dequant, bit-exact against the oracle's fp16 image
    {
        Tensor Wh;
        c.dequant(W, Wh);
        CHECK(Wh.dtype == Dtype::FP16 && Wh.rows == OUT && Wh.cols == IN && Wh.device == dev);
        bt::sync_all();
        std::vector<uint16_t> got((size_t)OUT * IN), want((size_t)OUT * IN);
        Wh.copy_to_host_fp16(got.data());
        oracle_dequant_16(c.fmt, Wb.data(), OUT, IN, 1, want.data());
        CHECK(got == want);
        Tensor W32 = Tensor::empty_on(dev, OUT, IN, Dtype::FP32);  // a pre-sized FP32 destination is kept
        c.dequant(W, W32);
        CHECK(W32.dtype == Dtype::FP32);
        std::vector<float> g32 = W32.to_host_vector(), w32((size_t)OUT * IN);
        oracle_dequant_f32(c.fmt, Wb.data(), OUT, IN, w32.data());
        CHECK(!std::memcmp(g32.data(), w32.data(), g32.size() * 4));
    }
    // B/C: GEMV with FP16 activations (the reference contract), with and without bias
    std::vector<float> xf(IN), bf(OUT);
    for (auto& v : xf) v = frand(-0.3f, 0.3f);
    for (auto& v : bf) v = frand(-0.1f, 0.1f);
    std::vector<uint16_t> xh(IN), bh(OUT);
    for (int i = 0; i < IN; ++i) { xh[i] = bt::fp32_to_fp16_bits(xf[i]); xf[i] = bt::fp16_bits_to_fp32(xh[i]); }
    for (int i = 0; i < OUT; ++i) { bh[i] = bt::fp32_to_fp16_bits(bf[i]); bf[i] = bt::fp16_bits_to_fp32(bh[i]); }
    std::vector<float> y_ref(OUT), yb_ref(OUT);
    oracle_matmul(c.fmt, Wb.data(), xf.data(), nullptr, y_ref.data(), nullptr, 1, OUT, IN, 1);
    oracle_matmul(c.fmt, Wb.data(), xf.data(), bf.data(), yb_ref.data(), nullptr, 1, OUT, IN, 1);
    {
        Tensor x = Tensor::from_host_fp16_on(dev, xh.data(), IN, 1), y;
        c.gemv(W, nullptr, x, y);
        CHECK(y.dtype == Dtype::FP16 && y.rows == OUT && y.cols == 1);
        bt::sync_all();
        std::vector<uint16_t> got = y.to_host_vector_fp16();
        bool within = true;
        for (int r = 0; r < OUT; ++r)
            if (std::fabs(bt::fp16_bits_to_fp32(got[r]) - y_ref[r]) > 3e-2f + 5e-2f * std::fabs(y_ref[r])) within = false;
        CHECK(within);
        Tensor bias = Tensor::from_host_fp16_on(dev, bh.data(), OUT, 1), yb;
        c.gemv(W, &bias, x, yb);
        got = yb.to_host_vector_fp16();
        within = true;
        for (int r = 0; r < OUT; ++r)
            if (std::fabs(bt::fp16_bits_to_fp32(got[r]) - yb_ref[r]) > 3e-2f + 5e-2f * std::fabs(yb_ref[r])) within = false;
        CHECK(within);
        // FP32 activations -> FP32 output, tight bound
        Tensor x32 = Tensor::from_host_on(dev, xf.data(), IN, 1), y32;
        c.gemv(W, nullptr, x32, y32);
        CHECK(y32.dtype == Dtype::FP32);
        CHECK(rel_l2(y32.to_host_vector(), y_ref) < 2e-3);
        // argument errors, with the reference's wording
        Tensor xi = Tensor::zeros_on(dev, IN, 1, Dtype::INT8), ybad;
        CHECK(throws_with([&] { c.gemv(W, nullptr, xi, ybad); }, "x must be FP16"));
        Tensor xs = Tensor::zeros_on(dev, IN / 2, 1, Dtype::FP16);
        CHECK(throws_with([&] { c.gemv(W, nullptr, xs, ybad); }, "x shape must be (in, 1)"));
        Tensor b2 = Tensor::zeros_on(dev, OUT + 1, 1, Dtype::FP16);
        CHECK(throws_with([&] { c.gemv(W, &b2, x, ybad); }, "bias shape must be (out, 1)"));
        Tensor b3 = Tensor::zeros_on(dev, OUT, 1, Dtype::FP32);
        CHECK(throws_with([&] { c.gemv(W, &b3, x, ybad); }, "bias must be FP16"));
        Tensor wrong = Tensor::zeros_on(dev, 4, IN, Dtype::FP16);
        CHECK(throws_with([&] { c.gemv(wrong, nullptr, x, ybad); }, "W must be Dtype::"));
        Tensor host_x = Tensor::zeros_on(Device::CPU, IN, 1, Dtype::FP16);
        CHECK(throws_with([&] { c.gemv(W, nullptr, host_x, ybad); }, "is on CPU but the op resolved to CUDA"));
    }
    // D/E/F/G: batched; the tensor-core counter tells which path ran
    for (int B : {4, 2, 16, 32}) {
        std::vector<float> Xf((size_t)B * IN);
        std::vector<uint16_t> Xh((size_t)B * IN);
        for (size_t i = 0; i < Xf.size(); ++i) { Xh[i] = bt::fp32_to_fp16_bits(frand(-0.3f, 0.3f)); Xf[i] = bt::fp16_bits_to_fp32(Xh[i]); }
        std::vector<float> Yref((size_t)B * OUT);
        oracle_matmul(c.fmt, Wb.data(), Xf.data(), nullptr, Yref.data(), nullptr, B, OUT, IN, 2);
        Tensor X = Tensor::from_host_fp16_on(dev, Xh.data(), B, IN), Y;
        bt::sync_all();
        (void)c.tc_calls();
        c.batched(W, nullptr, X, Y);
        CHECK(Y.dtype == Dtype::FP16 && Y.rows == B && Y.cols == OUT);
        bt::sync_all();
        const unsigned long long calls = c.tc_calls();
        std::vector<uint16_t> got = Y.to_host_vector_fp16();
        // random scale bytes make large outputs, so the bound is the mixed one of the reference's
        // prefill test (tests/test_quant_prefill_parity.cpp:133-145): |e| <= 3e-2 + 5e-2 * |ref|
        float max_abs = 0;
        bool within = true;
        for (size_t i = 0; i < got.size(); ++i) {
            const float e = std::fabs(bt::fp16_bits_to_fp32(got[i]) - Yref[i]);
            max_abs = std::fmax(max_abs, e);
            if (e > 3e-2f + 5e-2f * std::fabs(Yref[i])) within = false;
        }
        std::printf("  batched B=%d tc_calls=%llu max_abs=%g\n", B, calls, max_abs);
        CHECK(within);
        if (B <= 8) CHECK(calls == 0);  // small batches stream the weight once through the decode GEMV
        else CHECK(calls > 0);          // prefill batches run on the tensor cores
        Tensor bias_row = Tensor::zeros_on(dev, 1, OUT, Dtype::FP16), Yb;  // (1,out) bias is accepted for batched
        c.batched(W, &bias_row, X, Yb);
        Tensor Xbad = Tensor::zeros_on(dev, B, IN / 2, Dtype::FP16);
        CHECK(throws_with([&] { c.batched(W, nullptr, Xbad, Yb); }, "shape mismatch (W.cols != X.cols)"));
    }
}

static void test_gpu_large_rows_and_views() {
    std::printf("test_gpu_large_rows_and_views\n");
    // H: 70 000 one-block Q8_0 rows: the full decode equals the decode of the two halves
    const int R = 70000, IN = 32;
    FmtCase c{"q8_0", B200Q_FMT_Q8_0, Dtype::Q8_0, 32, 34, nullptr, nullptr, nullptr, nullptr};
    std::vector<uint8_t> Wb = make_blocks(c, R, IN);
    Tensor W = Tensor::from_raw_bytes_on(Device::CUDA, Wb.data(), R, IN, Dtype::Q8_0, Wb.size());
    Tensor full, a, b;
    bt::dequant_q8_0_to_fp16(W, full);
    const int H0 = R / 2;
    Tensor W0 = Tensor::from_raw_bytes_on(Device::CUDA, Wb.data(), H0, IN, Dtype::Q8_0, (size_t)H0 * 34);
    Tensor W1 = Tensor::from_raw_bytes_on(Device::CUDA, Wb.data() + (size_t)H0 * 34, R - H0, IN, Dtype::Q8_0, (size_t)(R - H0) * 34);
    bt::dequant_q8_0_to_fp16(W0, a);
    bt::dequant_q8_0_to_fp16(W1, b);
    bt::sync_all();
    std::vector<uint16_t> g = full.to_host_vector_fp16(), ga = a.to_host_vector_fp16(), gb = b.to_host_vector_fp16();
    ga.insert(ga.end(), gb.begin(), gb.end());
    CHECK(g == ga);
    // an unsized output adopts the op's device; resize keeps the pointer for graph replay
    Tensor x = Tensor::zeros_on(Device::CUDA, IN, 1, Dtype::FP16), y;
    bt::linear_forward_q8_0_fp16(W0, nullptr, x, y);
    void* p = y.data;
    bt::linear_forward_q8_0_fp16(W0, nullptr, x, y);
    CHECK(y.device == Device::CUDA && y.data == p && y.rows == H0);
}

static void test_gpu_group_op() {
    std::printf("test_gpu_group_op\n");
    // three Q4_K matrices against one x in one launch == three linear_forward_q4k_fp16 calls
    FmtCase c{"q4k", B200Q_FMT_Q4_K, Dtype::Q4_K, 256, 144, nullptr, nullptr, nullptr, nullptr};
    const int IN = 512, outs[3] = {96, 40, 250};
    std::vector<Tensor> W(3), yg(3), ys(3);
    for (int i = 0; i < 3; ++i) {
        std::vector<uint8_t> b = make_blocks(c, outs[i], IN);
        b[7 * i] ^= 0x11;  // make the three matrices differ
        W[i] = Tensor::from_raw_bytes_on(Device::CUDA, b.data(), outs[i], IN, Dtype::Q4_K, b.size());
    }
    std::vector<float> xh(IN);
    for (int i = 0; i < IN; ++i) xh[i] = 0.01f * (float)((i * 37) % 61 - 30);
    Tensor x = Tensor::from_host_on(Device::CUDA, xh.data(), IN, 1);
    const Tensor* Wp[3] = {&W[0], &W[1], &W[2]};
    Tensor* yp[3] = {&yg[0], &yg[1], &yg[2]};
    bt::linear_forward_group_fp16(Wp, nullptr, 3, x, yp);
    for (int i = 0; i < 3; ++i) bt::linear_forward_q4k_fp16(W[i], nullptr, x, ys[i]);
    bt::sync_all();
    for (int i = 0; i < 3; ++i) {
        CHECK(yg[i].rows == outs[i] && yg[i].cols == 1 && yg[i].dtype == Dtype::FP32 && yg[i].device == Device::CUDA);
        CHECK(yg[i].to_host_vector() == ys[i].to_host_vector());
    }
    // a matrix with another number of columns is refused with the op's name
    std::vector<uint8_t> b2 = make_blocks(c, 16, 256);
    Tensor W2 = Tensor::from_raw_bytes_on(Device::CUDA, b2.data(), 16, 256, Dtype::Q4_K, b2.size());
    const Tensor* bad[2] = {&W[0], &W2};
    Tensor t0, t1;
    Tensor* yb[2] = {&t0, &t1};
    bool threw = false;
    try {
        bt::linear_forward_group_fp16(bad, nullptr, 2, x, yb);
    } catch (const std::runtime_error& e) {
        threw = std::string(e.what()).find("brotensor: linear_forward_group_fp16:") == 0;
    }
    CHECK(threw);
}

static void test_gpu_repack_weights() {
    std::printf("test_gpu_repack_weights\n");
    // a Q6_K weight regrouped in place gives every op's raw-layout bits; views, copies and freed
    // storage follow the record; unpack restores the GGUF bytes
    FmtCase c{"q6k", B200Q_FMT_Q6_K, Dtype::Q6_K, 256, 210, nullptr, nullptr, nullptr, nullptr};
    const int OUT = 72, IN = 4096;
    std::vector<uint8_t> blocks = make_blocks(c, OUT, IN);
    Tensor W = Tensor::from_raw_bytes_on(Device::CUDA, blocks.data(), OUT, IN, Dtype::Q6_K, blocks.size());
    std::vector<float> xh(IN);
    for (int i = 0; i < IN; ++i) xh[i] = 0.02f * (float)((i * 53) % 47 - 23);
    Tensor x = Tensor::from_host_on(Device::CUDA, xh.data(), IN, 1);
    Tensor y_raw, d_raw, y_pk, d_pk, y_view, y_clone;
    bt::linear_forward_q6k_fp16(W, nullptr, x, y_raw);
    bt::dequant_q6k_to_fp16(W, d_raw);
    CHECK(!bt::is_repacked(W));
    CHECK(bt::repack_weights(W) && bt::is_repacked(W));
    std::vector<uint8_t> moved(blocks.size());
    {
        // the regrouped bytes never reach host code by accident: byte copies to the host are refused
        int refused = 0;
        try {
            W.copy_raw_to_host(moved.data());
        } catch (const std::runtime_error& e) {
            refused += std::string(e.what()).find("regrouped device layout") != std::string::npos;
        }
        try {
            Tensor onhost = W.to(Device::CPU);
        } catch (const std::runtime_error& e) {
            refused += std::string(e.what()).find("regrouped device layout") != std::string::npos;
        }
        CHECK(refused == 2);
    }
    bt::linear_forward_q6k_fp16(W, nullptr, x, y_pk);
    bt::dequant_q6k_to_fp16(W, d_pk);
    CHECK(y_pk.to_host_vector() == y_raw.to_host_vector());
    CHECK(d_pk.to_host_vector_fp16() == d_raw.to_host_vector_fp16());
    // rows [24, 72) as a non-owning view (what a row-sharded head passes)
    const std::size_t row_bytes = blocks.size() / OUT;
    Tensor Wv = Tensor::view(Device::CUDA, static_cast<char*>(W.data) + 24 * row_bytes, OUT - 24, IN, Dtype::Q6_K);
    CHECK(bt::is_repacked(Wv));
    bt::linear_forward_q6k_fp16(Wv, nullptr, x, y_view);
    {
        const std::vector<float> a = y_view.to_host_vector(), b = y_raw.to_host_vector();
        CHECK(std::vector<float>(b.begin() + 24, b.end()) == a);
    }
    bool threw = false;
    try {
        bt::repack_weights(Wv);  // already regrouped: fine
        bt::unpack_weights(Wv);  // a view may not change the layout
    } catch (const std::runtime_error& e) {
        threw = std::string(e.what()).find("brotensor: unpack_weights:") == 0;
    }
    CHECK(threw);
    Tensor Wc = W.clone();
    CHECK(bt::is_repacked(Wc));
    bt::linear_forward_q6k_fp16(Wc, nullptr, x, y_clone);
    CHECK(y_clone.to_host_vector() == y_raw.to_host_vector());
    bt::unpack_weights(W);
    CHECK(!bt::is_repacked(W) && bt::is_repacked(Wc));
    W.copy_raw_to_host(moved.data());
    CHECK(moved == blocks);
    // formats and shapes without a regrouped form
    FmtCase c4{"q4k", B200Q_FMT_Q4_K, Dtype::Q4_K, 256, 144, nullptr, nullptr, nullptr, nullptr};
    std::vector<uint8_t> b4 = make_blocks(c4, 8, 512);
    Tensor W4 = Tensor::from_raw_bytes_on(Device::CUDA, b4.data(), 8, 512, Dtype::Q4_K, b4.size());
    CHECK(!bt::repack_weights(W4) && !bt::is_repacked(W4));
    std::vector<uint8_t> b6 = make_blocks(c, 8, 768);
    Tensor W6 = Tensor::from_raw_bytes_on(Device::CUDA, b6.data(), 8, 768, Dtype::Q6_K, b6.size());
    CHECK(!bt::repack_weights(W6) && !bt::is_repacked(W6));
    bt::sync_all();
}

static void test_gpu_swiglu_op() {
    std::printf("test_gpu_swiglu_op\n");
    // silu(W_gate x) * (W_up x) in one launch against the two GEMVs and the gate on the host
    FmtCase c{"q4k", B200Q_FMT_Q4_K, Dtype::Q4_K, 256, 144, nullptr, nullptr, nullptr, nullptr};
    const int OUT = 200, IN = 1024;
    std::vector<uint8_t> bg = make_blocks(c, OUT, IN), bu = make_blocks(c, OUT, IN);
    for (std::size_t i = 0; i < bu.size(); i += 7) bu[i] ^= 0x5a;
    Tensor Wg = Tensor::from_raw_bytes_on(Device::CUDA, bg.data(), OUT, IN, Dtype::Q4_K, bg.size());
    Tensor Wu = Tensor::from_raw_bytes_on(Device::CUDA, bu.data(), OUT, IN, Dtype::Q4_K, bu.size());
    std::vector<float> xh(IN);
    for (int i = 0; i < IN; ++i) xh[i] = 0.03f * (float)((i * 29) % 41 - 20);
    Tensor x = Tensor::from_host_on(Device::CUDA, xh.data(), IN, 1);
    Tensor y, g, u;
    bt::linear_forward_swiglu_fp16(Wg, Wu, x, y);
    bt::linear_forward_q4k_fp16(Wg, nullptr, x, g);
    bt::linear_forward_q4k_fp16(Wu, nullptr, x, u);
    bt::sync_all();
    CHECK(y.rows == OUT && y.cols == 1 && y.dtype == Dtype::FP32);
    const std::vector<float> yv = y.to_host_vector(), gv = g.to_host_vector(), uv = u.to_host_vector();
    double worst = 0;
    for (int i = 0; i < OUT; ++i) {
        const double want = (double)gv[i] / (1.0 + std::exp(-(double)gv[i])) * (double)uv[i];
        worst = std::max(worst, std::fabs((double)yv[i] - want) / (std::fabs(want) + 1e-30));
    }
    CHECK(worst < 4e-6);
    bool threw = false;
    try {
        Tensor W2 = Tensor::from_raw_bytes_on(Device::CUDA, bu.data(), OUT / 2, IN, Dtype::Q4_K, bu.size() / 2);
        bt::linear_forward_swiglu_fp16(Wg, W2, x, y);
    } catch (const std::runtime_error& e) {
        threw = std::string(e.what()).find("brotensor: linear_forward_swiglu_fp16:") == 0;
    }
    CHECK(threw);
}

static void test_gpu_group_rmsnorm_op() {
    std::printf("test_gpu_group_rmsnorm_op\n");
    // two Q4_K matrices on rms_norm(x) * gamma in one launch == the grouped op on the host-normalised vector
    FmtCase c{"q4k", B200Q_FMT_Q4_K, Dtype::Q4_K, 256, 144, nullptr, nullptr, nullptr, nullptr};
    const int IN = 1024, outs[2] = {80, 33};
    const float eps = 1e-5f;
    std::vector<Tensor> W(2), yf(2), yr(2);
    for (int i = 0; i < 2; ++i) {
        std::vector<uint8_t> b = make_blocks(c, outs[i], IN);
        b[11 * (i + 1)] ^= 0x21;
        W[i] = Tensor::from_raw_bytes_on(Device::CUDA, b.data(), outs[i], IN, Dtype::Q4_K, b.size());
    }
    std::vector<float> xh(IN), gh(IN), xn(IN);
    double ss = 0;
    for (int i = 0; i < IN; ++i) {
        xh[i] = 0.05f * (float)((i * 31) % 53 - 26);
        gh[i] = 1.0f + 0.01f * (float)(i % 17);
        ss += (double)xh[i] * xh[i];
    }
    const double rr = 1.0 / std::sqrt(ss / IN + eps);
    for (int i = 0; i < IN; ++i) xn[i] = (float)(xh[i] * rr * gh[i]);
    Tensor x = Tensor::from_host_on(Device::CUDA, xh.data(), IN, 1), g = Tensor::from_host_on(Device::CUDA, gh.data(), IN, 1);
    Tensor xnd = Tensor::from_host_on(Device::CUDA, xn.data(), IN, 1);
    const Tensor* Wp[2] = {&W[0], &W[1]};
    Tensor* yfp[2] = {&yf[0], &yf[1]};
    Tensor* yrp[2] = {&yr[0], &yr[1]};
    bt::linear_forward_group_rmsnorm_fp16(Wp, 2, x, g, eps, yfp);
    bt::linear_forward_group_fp16(Wp, nullptr, 2, xnd, yrp);
    bt::sync_all();
    for (int i = 0; i < 2; ++i) {
        const std::vector<float> a = yf[i].to_host_vector(), b = yr[i].to_host_vector();
        CHECK((int)a.size() == outs[i]);
        double num = 0, den = 0;
        for (std::size_t k = 0; k < a.size(); ++k) { num += ((double)a[k] - b[k]) * ((double)a[k] - b[k]); den += (double)b[k] * b[k]; }
        CHECK(std::sqrt(num / (den + 1e-30)) < 2e-4);
    }
    bool threw = false;
    try {
        Tensor g2 = Tensor::from_host_on(Device::CUDA, gh.data(), IN / 2, 1);
        bt::linear_forward_group_rmsnorm_fp16(Wp, 2, x, g2, eps, yfp);
    } catch (const std::runtime_error& e) {
        threw = std::string(e.what()).find("brotensor: linear_forward_group_rmsnorm_fp16:") == 0;
    }
    CHECK(threw);
}

// Q4_0 and Q5_K (formats brotensor's loader carries without ops) through the public ops, and the
// quantized embedding lookup that brotensor refuses (tests/test_embedding_extra_parity.cpp:141-154
// pins that refusal; here the same call returns the rows' exact decode).
static void test_gpu_extra_formats_and_embedding() {
    std::printf("test_gpu_extra_formats_and_embedding\n");
    const Device dev = Device::CUDA;
    struct Extra {
        FmtCase c;
    } extras[] = {
        {{"q4_0", B200Q_FMT_Q4_0, Dtype::Q4_0, 32, 18, bt::dequant_q4_0_to_fp16, bt::linear_forward_q4_0_fp16, bt::linear_forward_batched_q4_0_fp16, nullptr}},
        {{"q5k", B200Q_FMT_Q5_K, Dtype::Q5_K, 256, 176, bt::dequant_q5k_to_fp16, bt::linear_forward_q5k_fp16, bt::linear_forward_batched_q5k_fp16, nullptr}},
    };
    for (const auto& e : extras) {
        const FmtCase& c = e.c;
        const int OUT = 96, IN = 512, B = 16;
        std::vector<uint8_t> Wb = make_blocks(c, OUT, IN);
        if (c.fmt == B200Q_FMT_Q4_0 || c.fmt == B200Q_FMT_Q5_K) {  // their fp16 fields sit at the block's start
            for (size_t i = 0; i < Wb.size() / c.bytes; ++i) {
                uint8_t* p = &Wb[i * c.bytes];
                auto put = [&](int off, float f) { const uint16_t h = bt::fp32_to_fp16_bits(f); p[off] = h & 0xFF; p[off + 1] = h >> 8; };
                put(0, 0.02f * frand(0.5f, 1.5f));
                if (c.fmt == B200Q_FMT_Q5_K) put(2, 0.008f * frand(0.5f, 1.5f));
            }
        }
        Tensor W = Tensor::empty_on(dev, OUT, IN, c.dt);
        cudaMemcpy(W.data, Wb.data(), Wb.size(), cudaMemcpyHostToDevice);
        Tensor Wh;
        c.dequant(W, Wh);
        CHECK(Wh.dtype == Dtype::FP16 && Wh.rows == OUT && Wh.cols == IN);
        std::vector<uint16_t> got((size_t)OUT * IN), want((size_t)OUT * IN);
        Wh.copy_to_host_fp16(got.data());
        oracle_dequant_16(c.fmt, Wb.data(), OUT, IN, 1, want.data());
        CHECK(got == want);
        std::vector<float> xf(IN), Xf((size_t)B * IN), y_ref(OUT), Y_ref((size_t)B * OUT);
        for (auto& v : xf) v = frand(-0.3f, 0.3f);
        for (auto& v : Xf) v = frand(-0.3f, 0.3f);
        oracle_matmul(c.fmt, Wb.data(), xf.data(), nullptr, y_ref.data(), nullptr, 1, OUT, IN, 1);
        oracle_matmul(c.fmt, Wb.data(), Xf.data(), nullptr, Y_ref.data(), nullptr, B, OUT, IN, 2);
        Tensor x = Tensor::from_host_on(dev, xf.data(), IN, 1), y;
        c.gemv(W, nullptr, x, y);
        CHECK(y.dtype == Dtype::FP32 && y.rows == OUT && y.cols == 1);
        CHECK(rel_l2(y.to_host_vector(), y_ref) < 2e-3);
        Tensor X = Tensor::from_host_on(dev, Xf.data(), B, IN), Y;
        c.batched(W, nullptr, X, Y);
        CHECK(Y.rows == B && Y.cols == OUT);
        CHECK(rel_l2(Y.to_host_vector(), Y_ref) < 2e-3);
        Tensor wrong = Tensor::zeros_on(dev, 4, IN, Dtype::FP16);
        CHECK(throws_with([&] { c.gemv(wrong, nullptr, x, y); }, "W must be Dtype::"));
    }
    // quantized embedding lookup
    {
        const FmtCase q4{"q4k", B200Q_FMT_Q4_K, Dtype::Q4_K, 256, 144, nullptr, nullptr, nullptr, nullptr};
        const int V = 300, D = 512, B = 6;
        const std::vector<uint8_t> Tb = make_blocks(q4, V, D);
        Tensor table = Tensor::empty_on(dev, V, D, Dtype::Q4_K);
        cudaMemcpy(table.data, Tb.data(), Tb.size(), cudaMemcpyHostToDevice);
        const int32_t idx_h[B] = {7, 0, 299, 7, -3, 300};
        int32_t* d_idx = nullptr;
        cudaMalloc(reinterpret_cast<void**>(&d_idx), sizeof(idx_h));
        cudaMemcpy(d_idx, idx_h, sizeof(idx_h), cudaMemcpyHostToDevice);
        Tensor out;
        bt::embedding_lookup_forward(table, d_idx, B, out);
        CHECK(out.rows == B && out.cols == D && out.dtype == Dtype::FP16 && out.device == dev);
        std::vector<uint16_t> got((size_t)B * D), full((size_t)V * D);
        out.copy_to_host_fp16(got.data());
        oracle_dequant_16(B200Q_FMT_Q4_K, Tb.data(), V, D, 1, full.data());
        bool ok = true, zeros = true;
        for (int b = 0; b < B; ++b)
            for (int j = 0; j < D; ++j) {
                if (idx_h[b] >= 0 && idx_h[b] < V) ok = ok && got[(size_t)b * D + j] == full[(size_t)idx_h[b] * D + j];
                else zeros = zeros && got[(size_t)b * D + j] == 0;
            }
        CHECK(ok);
        CHECK(zeros);  // indices outside the table give rows of zeros
        Tensor out32 = Tensor::empty_on(dev, B, D, Dtype::FP32);
        bt::embedding_lookup_forward(table, d_idx, B, out32);
        CHECK(out32.dtype == Dtype::FP32);
        Tensor dense = Tensor::zeros_on(dev, V, D, Dtype::FP16);
        CHECK(throws_with([&] { bt::embedding_lookup_forward(dense, d_idx, B, out); }, "table dtype must be"));
        CHECK(throws_with([&] { bt::embedding_lookup_forward(table, nullptr, B, out); }, "null index"));
        Tensor none;
        bt::embedding_lookup_forward(table, d_idx, 0, none);
        CHECK(none.rows == 0 && none.cols == D);
        cudaFree(d_idx);
    }
}

int main(int argc, char** argv) {
    const std::string mode = argc > 1 ? argv[1] : "cpu";
    bt::init();
    if (mode == "cpu") {
        test_cpu_tensor_and_dispatch();
        test_cpu_gguf();
    } else {
        if (!bt::is_available(Device::CUDA)) {
            std::printf("no CUDA device available - skipping\n");
            return 0;
        }
        const FmtCase cases[] = {
            {"q4k", B200Q_FMT_Q4_K, Dtype::Q4_K, 256, 144, bt::dequant_q4k_to_fp16, bt::linear_forward_q4k_fp16,
             bt::linear_forward_batched_q4k_fp16, brotensor_q4k_wmma_calls_consume},
            {"q6k", B200Q_FMT_Q6_K, Dtype::Q6_K, 256, 210, bt::dequant_q6k_to_fp16, bt::linear_forward_q6k_fp16,
             bt::linear_forward_batched_q6k_fp16, brotensor_q6k_wmma_calls_consume},
            {"q8_0", B200Q_FMT_Q8_0, Dtype::Q8_0, 32, 34, bt::dequant_q8_0_to_fp16, bt::linear_forward_q8_0_fp16,
             bt::linear_forward_batched_q8_0_fp16, brotensor_q8_0_wmma_calls_consume},
        };
        for (const auto& c : cases) run_fmt(c);
        test_gpu_large_rows_and_views();
        test_gpu_group_op();
        test_gpu_repack_weights();
        test_gpu_swiglu_op();
        test_gpu_group_rmsnorm_op();
        test_gpu_extra_formats_and_embedding();
        int st = 0;
        CHECK(b200q_device_status(&st) == B200Q_OK && st == 0);
    }
    std::printf("%s (%d failures)\n", g_failures ? "FAILED" : "OK", g_failures);
    return g_failures ? 1 : 0;
}

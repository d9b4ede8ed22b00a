// Backend bring-up and runtime policy (brotensor src/init.cpp:68-120, 221-225;
// src/cuda/register.cu:77-157; src/cuda/runtime.cu:41-74). The CPU allocator registers
// itself at static-init time with no ops (brotensor's CPU backend has no quant ops
// either, so they report "not implemented on CPU"); init() probes CUDA, enables peer
// access between all device pairs, sets up the async memory pools and registers the
// CUDA tables.
#include "brotensor_b200/runtime.h"

#include <cuda_runtime_api.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <stdexcept>

#include "brotensor_b200/detail/dispatch.h"

namespace brotensor_b200 {

namespace detail {
void fill_cuda_tables(OpsVTable& ops, AllocVTable& alloc);  // cuda_backend.cpp
}

namespace {

// ---- CPU allocator table ----
void* cpu_alloc(std::size_t n, int) { return n ? std::malloc(n) : nullptr; }
void cpu_free(void* p, int) { std::free(p); }
void cpu_copy(void* d, const void* s, std::size_t n, int) { std::memcpy(d, s, n); }
void cpu_peer(void* d, int, const void* s, int, std::size_t n) { std::memcpy(d, s, n); }
void cpu_zero(void* d, std::size_t n, int) { std::memset(d, 0, n); }
void cpu_sync(int) {}

struct CpuRegistrar {
    CpuRegistrar() {
        detail::OpsVTable ops{};  // every quant slot stays null on CPU
        detail::AllocVTable a{};
        a.alloc = cpu_alloc; a.free = cpu_free;
        a.memcpy_h2d = cpu_copy; a.memcpy_d2h = cpu_copy; a.memcpy_d2d = cpu_copy;
        a.memcpy_h2d_async = cpu_copy; a.memcpy_d2h_async = cpu_copy;
        a.memcpy_peer = cpu_peer; a.memset_zero = cpu_zero; a.sync = cpu_sync;
        detail::register_backend(DeviceType::CPU, ops, a);
    }
} g_cpu_registrar;

std::mutex g_init_mu;
bool g_inited = false;
Device g_default = Device::CPU;
bool g_default_set = false;
thread_local bool t_has_override = false;
thread_local Device t_override = Device::CPU;

constexpr int kMaxStreams = 16;
thread_local cudaStream_t t_streams[kMaxStreams] = {nullptr};
int stream_index(int dev) {
    if (dev < 0) {
        int d = 0;
        if (cudaGetDevice(&d) != cudaSuccess) d = 0;
        dev = d;
    }
    return (dev >= 0 && dev < kMaxStreams) ? dev : 0;
}

Device parse_device_env(const char* s) {
    if (!s) return Device::CPU;
    if (!std::strcmp(s, "cpu") || !std::strcmp(s, "CPU")) return Device::CPU;
    if (!std::strncmp(s, "cuda", 4) || !std::strncmp(s, "CUDA", 4)) {
        int idx = 0;
        if (s[4] == ':') idx = std::atoi(s + 5);
        return Device::cuda(idx);
    }
    return Device::CPU;
}

}  // namespace

void init() {
    std::lock_guard<std::mutex> lk(g_init_mu);
    if (g_inited) return;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        (void)cudaGetLastError();
        n = 0;
    }
    if (n > 0) {
        int prev = 0;
        cudaGetDevice(&prev);
        for (int i = 0; i < n; ++i) {
            cudaSetDevice(i);
            cudaMemPool_t pool;
            if (cudaDeviceGetDefaultMemPool(&pool, i) == cudaSuccess) {
                unsigned long long keep = ~0ull;  // never hand cached blocks back on sync
                cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
            }
            for (int j = 0; j < n; ++j) {
                if (i == j) continue;
                int can = 0;
                if (cudaDeviceCanAccessPeer(&can, i, j) == cudaSuccess && can) {
                    const cudaError_t e = cudaDeviceEnablePeerAccess(j, 0);
                    if (e != cudaSuccess) (void)cudaGetLastError();  // already enabled is fine
                }
            }
        }
        cudaSetDevice(prev);
        detail::OpsVTable ops{};
        detail::AllocVTable alloc{};
        detail::fill_cuda_tables(ops, alloc);
        detail::set_cuda_device_count(n);
        detail::register_backend(DeviceType::CUDA, ops, alloc);
    }
    if (!g_default_set) {
        const Device want = parse_device_env(std::getenv("BROTENSOR_DEFAULT_DEVICE"));
        if (want.is_cuda() && want.index < n) g_default = want;
    }
    g_inited = true;
}

void shutdown() {
    std::lock_guard<std::mutex> lk(g_init_mu);
    g_inited = false;
}

int cuda_device_count() { return detail::get_cuda_device_count(); }
bool is_available(Device d) { return detail::is_registered(d); }
std::vector<Device> available_devices() {
    std::vector<Device> v{Device::CPU};
    for (int i = 0; i < cuda_device_count(); ++i) v.push_back(Device::cuda(i));
    return v;
}
Device default_device() { return t_has_override ? t_override : g_default; }
void set_default_device(Device d) {
    if (!is_available(d)) throw std::runtime_error("brotensor: set_default_device: device " + to_string(d) + " is not available");
    g_default = d;
    g_default_set = true;
}
DeviceScope::DeviceScope(Device d) : prev_(default_device()) {
    if (!is_available(d)) throw std::runtime_error("brotensor: DeviceScope: device " + to_string(d) + " is not available");
    t_override = d;
    t_has_override = true;
}
DeviceScope::~DeviceScope() { t_override = prev_; }

void sync(Device d) {
    if (!is_available(d)) return;
    detail::alloc_for(d).sync(d.index);
}
void sync_all() {
    for (Device d : available_devices()) sync(d);
}
bool device_mem_info(Device d, std::size_t& free_bytes, std::size_t& total_bytes) {
    if (!is_available(d)) return false;
    const auto& a = detail::alloc_for(d);
    return a.mem_info && a.mem_info(&free_bytes, &total_bytes, d.index);
}
std::string device_product_name(Device d) {
    char buf[256] = "";
    if (is_available(d)) {
        const auto& a = detail::alloc_for(d);
        if (a.device_name && a.device_name(buf, sizeof(buf), d.index)) return buf;
    }
    return device_name(d);
}

void* cuda_current_stream(int dev) { return t_streams[stream_index(dev)]; }
void cuda_set_stream(void* stream, int dev) { t_streams[stream_index(dev)] = static_cast<cudaStream_t>(stream); }

}  // namespace brotensor_b200

// repack_weights / unpack_weights and the record of which storage is in the regrouped layout.
#include "brotensor_b200/repack.h"

#include <cstdint>
#include <map>
#include <mutex>
#include <shared_mutex>
#include <stdexcept>
#include <string>

#include "b200q.h"
#include "brotensor_b200/runtime.h"

namespace brotensor_b200 {

namespace {
std::shared_mutex g_mu;
std::map<std::uintptr_t, std::uintptr_t> g_ranges;  // begin -> end of regrouped storage

[[noreturn]] void rp_fail(const char* op, const std::string& why) {
    throw std::runtime_error(std::string("brotensor: ") + op + ": " + why);
}
int raw_fmt(Dtype dt) {
    switch (dt) {
        case Dtype::Q4_K: return B200Q_FMT_Q4_K;
        case Dtype::Q6_K: return B200Q_FMT_Q6_K;
        case Dtype::Q8_0: return B200Q_FMT_Q8_0;
        default: return -1;
    }
}
}  // namespace

namespace detail {
void mark_repacked(const void* data, std::size_t nbytes) {
    if (!data || !nbytes) return;
    std::unique_lock lk(g_mu);
    const auto b = reinterpret_cast<std::uintptr_t>(data);
    g_ranges[b] = b + nbytes;
}
void forget_repacked(const void* data) {
    if (!data) return;
    {
        std::shared_lock lk(g_mu);
        if (g_ranges.empty()) return;
    }
    std::unique_lock lk(g_mu);
    g_ranges.erase(reinterpret_cast<std::uintptr_t>(data));
}
bool repacked_ptr(const void* data) {
    if (!data) return false;
    std::shared_lock lk(g_mu);
    if (g_ranges.empty()) return false;
    const auto p = reinterpret_cast<std::uintptr_t>(data);
    auto it = g_ranges.upper_bound(p);
    if (it == g_ranges.begin()) return false;
    --it;
    return p < it->second;
}
}  // namespace detail

bool is_repacked(const Tensor& W) { return detail::repacked_ptr(W.data); }

bool repack_weights(Tensor& W) {
    const char* op = "repack_weights";
    const int fmt = raw_fmt(W.dtype);
    if (fmt < 0) rp_fail(op, "W must be Dtype::Q4_K, Q6_K or Q8_0");
    if (!W.device.is_cuda()) rp_fail(op, "W must live on a CUDA device");
    if (W.rows == 0 || W.cols == 0 || !W.data) return false;
    if (b200q_repacked_fmt(fmt, W.cols) == fmt) return false;
    if (is_repacked(W)) return true;
    if (!W.owns_storage()) rp_fail(op, "W must own its storage (repack the weight, not a view of it)");
    DeviceScope scope(W.device);
    const int rc = b200q_repack(fmt, W.data, W.data, W.rows, W.cols, cuda_current_stream(W.device.index));
    if (rc != B200Q_OK) rp_fail(op, b200q_last_error());
    detail::mark_repacked(W.data, W.bytes());
    return true;
}

void unpack_weights(Tensor& W) {
    const char* op = "unpack_weights";
    if (!is_repacked(W)) return;
    if (!W.owns_storage()) rp_fail(op, "W must own its storage");
    const int fmt = raw_fmt(W.dtype);
    DeviceScope scope(W.device);
    const int rc = b200q_unpack(fmt, W.data, W.data, W.rows, W.cols, cuda_current_stream(W.device.index));
    if (rc != B200Q_OK) rp_fail(op, b200q_last_error());
    detail::forget_repacked(W.data);
}

}  // namespace brotensor_b200

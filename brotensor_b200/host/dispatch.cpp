// Backend registry and operand-device resolution (brotensor src/dispatch.cpp:86-134,
// 151-186, 232-270): the first operand with storage picks the device, every other
// operand with storage must agree, the CUDA device is made current, and the backend's
// table is returned.
#include "brotensor_b200/detail/dispatch.h"

#include <cuda_runtime_api.h>

#include <stdexcept>
#include <string>

namespace brotensor_b200::detail {

namespace {
struct Slot {
    bool registered = false;
    OpsVTable ops;
    AllocVTable alloc;
};
Slot g_slots[3];
int g_cuda_count = 0;
Slot& slot(DeviceType t) { return g_slots[static_cast<int>(t)]; }
}  // namespace

void register_backend(DeviceType dt, const OpsVTable& ops, const AllocVTable& alloc) {
    Slot& s = slot(dt);
    s.ops = ops;
    s.alloc = alloc;
    s.registered = true;
}
bool is_registered(Device d) {
    if (!slot(d.type).registered) return false;
    if (d.type == DeviceType::CUDA) return d.index >= 0 && d.index < g_cuda_count;
    return d.index == 0;
}
const OpsVTable& ops_for(Device d) {
    if (!slot(d.type).registered)
        throw std::runtime_error(std::string("brotensor: backend ") + device_name(d) + " is not registered (call init())");
    return slot(d.type).ops;
}
const AllocVTable& alloc_for(Device d) {
    if (!slot(d.type).registered)
        throw std::runtime_error(std::string("brotensor: backend ") + device_name(d) + " is not registered (call init())");
    return slot(d.type).alloc;
}
void set_cuda_device_count(int n) { g_cuda_count = n; }
int get_cuda_device_count() { return g_cuda_count; }

const OpsVTable& dispatch_with_opts(const Tensor& a, std::initializer_list<const Tensor*> opts) {
    const Tensor* all[16];
    std::size_t n = 0;
    all[n++] = &a;
    for (const Tensor* t : opts)
        if (n < 16) all[n++] = t;
    Device dev = Device::CPU;
    bool found = false;
    for (std::size_t i = 0; i < n && !found; ++i)
        if (all[i] && all[i]->data) {
            dev = all[i]->device;
            found = true;
        }
    if (!found) dev = a.device;  // nothing has storage yet: keep operand 0's tag
    for (std::size_t i = 0; i < n; ++i)
        if (all[i] && all[i]->data && all[i]->device != dev)
            throw std::runtime_error("brotensor: dispatch: operand " + std::to_string(i) + " is on " +
                                     device_name(all[i]->device) + " but the op resolved to " + device_name(dev));
    if (dev.is_cuda()) cudaSetDevice(dev.index);
    return ops_for(dev);
}

void adopt_output(Tensor& t, Device d) {
    if (t.data == nullptr) t.device = d;
}

void throw_not_implemented(const char* op_name, Device d) {
    throw std::runtime_error(std::string("brotensor: ") + op_name + ": not implemented on " + device_name(d));
}

}  // namespace brotensor_b200::detail

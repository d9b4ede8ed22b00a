// Runtime policy of the b200 host layer: backend bring-up, default device, sync.
// Mirrors include/brotensor/runtime.h:18-117 for the calls the quant-matmul path
// and its tests use.
#pragma once

#include <cstddef>
#include <string>
#include <vector>

#include "tensor.h"

namespace brotensor_b200 {

// Probes CUDA and registers the backend tables. Idempotent and thread-safe. The CPU
// allocator is registered at static-init time, so host tensors work without init().
void init();
void shutdown();

Device default_device();
void set_default_device(Device d);
int cuda_device_count();
std::vector<Device> available_devices();
bool is_available(Device);

// RAII default-device override for the calling thread.
class DeviceScope {
public:
    explicit DeviceScope(Device d);
    ~DeviceScope();
    DeviceScope(const DeviceScope&) = delete;
    DeviceScope& operator=(const DeviceScope&) = delete;
private:
    Device prev_;
};

void sync(Device d);
void sync_all();
bool device_mem_info(Device d, std::size_t& free_bytes, std::size_t& total_bytes);
std::string device_product_name(Device d);

// The calling thread's current CUDA stream for device `dev` (-1 = current device);
// every op launches on it. nullptr is the legacy default stream.
void* cuda_current_stream(int dev = -1);
void cuda_set_stream(void* stream, int dev = -1);

}  // namespace brotensor_b200

// Per-device, thread-safe one-time set-up.  The library is called from several host threads for
// different devices (a framework's executor threads), so nothing here is cached in a plain global:
// every cached fact is keyed by the device ordinal and guarded by std::call_once.
#pragma once
#include <cuda_runtime.h>

#include <functional>
#include <mutex>

namespace b200wkv {

constexpr int kMaxDevices = 64;

inline int current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
    return dev;
}

// Number of SMs of the current device (148 on a B200; an SM-limited context reports its own count).
inline int sm_count_of_current_device() {
    static std::once_flag once[kMaxDevices];
    static int count[kMaxDevices];
    const int dev = current_device();
    if (dev < 0) return 148;
    std::call_once(once[dev], [dev]() {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        count[dev] = n;
    });
    return count[dev];
}

// Runs `setup` (returning a cudaError_t) once per device for one call site; later calls return the
// recorded result.  Use one DeviceOnce object (static storage) per thing that needs setting up.
struct DeviceOnce {
    std::once_flag once[kMaxDevices];
    cudaError_t result[kMaxDevices];
    bool ok(const std::function<cudaError_t()>& setup) {
        const int dev = current_device();
        if (dev < 0) return setup() == cudaSuccess;
        std::call_once(once[dev], [this, dev, &setup]() { result[dev] = setup(); });
        return result[dev] == cudaSuccess;
    }
};

}  // namespace b200wkv

// Per-device facts cached by the launchers: SM count and which kernels already had their
// dynamic shared-memory limit raised.  Function attributes belong to the current device's
// context, and a process may use several GPUs from several threads, so both are keyed by the
// device ordinal and guarded by a mutex.
#pragma once
#include <cuda_runtime.h>

#include <mutex>
#include <set>
#include <utility>

namespace natten {

constexpr int kMaxDynamicSmem = 232448;     // 227 KB: the most dynamic shared memory a CTA may ask for

struct DeviceCache {
    std::mutex mutex;
    int sms[64] = {0};
    std::set<std::pair<int, const void*>> smem_attr_done;
};
inline DeviceCache& device_cache()
{
    static DeviceCache c;
    return c;
}

inline int sm_count()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    DeviceCache& c = device_cache();
    std::lock_guard<std::mutex> lock(c.mutex);
    if (c.sms[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        c.sms[dev] = n;
    }
    return c.sms[dev];
}

// Function attributes belong to the current device's context: set the dynamic shared-memory
// limit of `kernel` once per device.
inline cudaError_t ensure_dynamic_smem(const void* kernel, int bytes)
{
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    DeviceCache& c = device_cache();
    std::lock_guard<std::mutex> lock(c.mutex);
    const auto key = std::make_pair(dev, kernel);
    if (c.smem_attr_done.count(key)) return cudaSuccess;
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (err == cudaSuccess) c.smem_attr_done.insert(key);
    return err;
}

} // namespace natten

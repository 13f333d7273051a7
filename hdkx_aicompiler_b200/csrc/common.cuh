// Shared host-side helpers for libkxc_b200: error reporting across the C ABI and launch checks.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <mutex>

#include "kxc_b200.h"

namespace kxc_b200 {

// Per-thread message behind kxc_b200_last_error(); the ABI itself only carries an int.
char* last_error_buffer();
constexpr size_t kLastErrorSize = 512;

inline int32_t fail(int32_t code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(last_error_buffer(), kLastErrorSize, fmt, ap);
    va_end(ap);
    return code;
}

// Device presence is checked once per process; every compute entry point goes through this so that a
// box without a Blackwell GPU fails loudly instead of computing somewhere else.
int32_t require_device();

inline int32_t check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(KXC_B200_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return KXC_B200_OK;
}

#define KXC_CUDA_TRY(expr)                                                                         \
    do {                                                                                           \
        cudaError_t _e = (expr);                                                                   \
        if (_e != cudaSuccess)                                                                     \
            return ::kxc_b200::fail(KXC_B200_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

#define KXC_TRY(expr)                     \
    do {                                  \
        int32_t _rc = (expr);             \
        if (_rc != KXC_B200_OK) return _rc; \
    } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int64_t conv_out_dim(int64_t in, int64_t k, int64_t s, int64_t p, int64_t d) {
    return (in + 2 * p - ((k - 1) * d + 1)) / s + 1;
}
inline int64_t pool_out_dim(int64_t in, int64_t k, int64_t s, int64_t p0, int64_t p1, bool ceil_mode) {
    const int64_t num = in + p0 + p1 - k;
    return ceil_mode ? ((num + s - 1) / s + 1) : (num / s + 1);
}

// Launch with optional programmatic dependent launch (the kernel must call sm100::pdl_wait() before it touches
// memory other kernels produce or consume) and an optional cluster of `cluster_x` CTAs.
// KXC_B200_PDL=0 in the environment launches everything fully serialized.
bool pdl_enabled();
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl,
                                 int cluster_x, Args&&... args) {
    cudaLaunchConfig_t lc = {};
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = (unsigned)cluster_x;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    if (pdl && pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    lc.gridDim = grid;
    lc.blockDim = block;
    lc.dynamicSmemBytes = smem;
    lc.stream = stream;
    lc.attrs = attr;
    lc.numAttrs = n;
    return cudaLaunchKernelEx(&lc, kernel, static_cast<KArgs>(args)...);
}

// Runs a set-up action once per CUDA device. Function attributes such as the dynamic shared-memory opt-in belong
// to the device that is current when they are set, so a process that drives several GPUs must repeat them on each.
class PerDeviceOnce {
  public:
    static constexpr int kMaxDevices = 64;
    // Calls `fn` (returning cudaError_t) the first time `device` is seen; later calls return that first result.
    // A failed action is retried on the next call.
    template <typename F>
    cudaError_t run(int device, F&& fn) {
        if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
        std::lock_guard<std::mutex> lock(mu_);
        if (!done_[device]) {
            const cudaError_t e = fn();
            if (e != cudaSuccess) return e;
            done_[device] = true;
        }
        return cudaSuccess;
    }

  private:
    std::mutex mu_;
    bool done_[kMaxDevices] = {};
};

// Opt-in to `bytes` of dynamic shared memory for `kernel` on the current device (once per device).
template <typename K>
inline int32_t smem_opt_in(PerDeviceOnce& once, K kernel, int bytes, int* device_out = nullptr) {
    int dev = 0;
    KXC_CUDA_TRY(cudaGetDevice(&dev));
    if (device_out) *device_out = dev;
    const cudaError_t e = once.run(dev, [&] {
        return cudaFuncSetAttribute(reinterpret_cast<const void*>(kernel), cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    });
    if (e != cudaSuccess)
        return fail(KXC_B200_ERR_CUDA, "cudaFuncSetAttribute(smem=%d) on device %d: %s", bytes, dev, cudaGetErrorString(e));
    return KXC_B200_OK;
}

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs; grids are sized in multiples of this

}  // namespace kxc_b200

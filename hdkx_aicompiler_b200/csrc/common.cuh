// Shared host-side helpers for libkxc_b200: error reporting across the C ABI and launch checks.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

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

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs; grids are sized in multiples of this

}  // namespace kxc_b200

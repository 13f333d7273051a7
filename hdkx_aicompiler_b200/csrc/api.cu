// C-ABI entry points of libkxc_b200 that validate a descriptor and dispatch to a kernel family.
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "conv_common.cuh"

namespace kxc_b200 {

char* last_error_buffer() {
    static thread_local char buf[kLastErrorSize] = {0};
    return buf;
}

bool pdl_enabled() {
    static const bool on = [] {
        const char* e = getenv("KXC_B200_PDL");
        return !(e != nullptr && e[0] == '0');
    }();
    return on;
}

int32_t require_device() {
    static std::once_flag once;
    static int32_t status = KXC_B200_ERR_NO_DEVICE;
    static char why[256] = "no CUDA device";
    std::call_once(once, [] {
        int count = 0;
        cudaError_t e = cudaGetDeviceCount(&count);
        if (e != cudaSuccess || count == 0) {
            snprintf(why, sizeof(why), "no CUDA device (%s); libkxc_b200 has no CPU fallback",
                     e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0");
            cudaGetLastError();
            return;
        }
        int dev = 0, major = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (major != 10) {
            snprintf(why, sizeof(why), "device %d has compute capability %d.x; the kernels are built for sm_100a only", dev, major);
            return;
        }
        status = KXC_B200_OK;
    });
    if (status != KXC_B200_OK) return fail(status, "%s", why);
    return KXC_B200_OK;
}

int32_t make_conv_dims(const kxc_b200_conv2d_desc* c, const char* name, ConvDims* d) {
    if (!c) return fail(KXC_B200_ERR_INVALID, "%s: null descriptor", name);
    if (c->n < 0 || c->c <= 0 || c->h <= 0 || c->w <= 0 || c->o <= 0 || c->kh <= 0 || c->kw <= 0 || c->stride_h <= 0 ||
        c->stride_w <= 0 || c->pad_h < 0 || c->pad_w < 0 || c->dilation_h <= 0 || c->dilation_w <= 0)
        return fail(KXC_B200_ERR_INVALID, "%s: bad shape/stride/padding/dilation", name);
    const int64_t OH = conv_out_dim(c->h, c->kh, c->stride_h, c->pad_h, c->dilation_h);
    const int64_t OW = conv_out_dim(c->w, c->kw, c->stride_w, c->pad_w, c->dilation_w);
    if (OH <= 0 || OW <= 0) return fail(KXC_B200_ERR_INVALID, "%s: empty output (%lld x %lld)", name, (long long)OH, (long long)OW);
    *d = ConvDims{c->n, c->c, c->h, c->w, c->o, c->kh, c->kw, c->stride_h, c->stride_w, c->pad_h, c->pad_w,
                  c->dilation_h, c->dilation_w, (int)OH, (int)OW};
    return KXC_B200_OK;
}

}  // namespace kxc_b200

using namespace kxc_b200;

extern "C" const char* kxc_b200_last_error(void) { return last_error_buffer(); }
extern "C" int32_t kxc_b200_abi_version(void) { return KXC_B200_ABI_VERSION; }
extern "C" int32_t kxc_b200_device_check(void) { return require_device(); }

// Host-only check of the once-per-device bookkeeping behind the shared-memory opt-in: the action must run exactly
// once for every device ordinal it is asked for, be retried after a failure, and refuse ordinals out of range.
extern "C" int32_t kxc_b200_selftest_per_device_once(void) {
    PerDeviceOnce once;
    int calls[PerDeviceOnce::kMaxDevices] = {0};
    auto run = [&](int dev, cudaError_t result) { return once.run(dev, [&] { ++calls[dev]; return result; }); };
    if (run(0, cudaSuccess) != cudaSuccess || run(1, cudaSuccess) != cudaSuccess || run(0, cudaSuccess) != cudaSuccess ||
        run(1, cudaSuccess) != cudaSuccess || run(63, cudaSuccess) != cudaSuccess)
        return fail(KXC_B200_ERR_INVALID, "per-device once: a valid device was refused");
    if (calls[0] != 1 || calls[1] != 1 || calls[63] != 1) return fail(KXC_B200_ERR_INVALID, "per-device once: action ran %d/%d/%d times", calls[0], calls[1], calls[63]);
    if (run(2, cudaErrorInvalidValue) != cudaErrorInvalidValue || run(2, cudaSuccess) != cudaSuccess || run(2, cudaSuccess) != cudaSuccess || calls[2] != 2)
        return fail(KXC_B200_ERR_INVALID, "per-device once: a failed action must be retried once, then remembered");
    if (run(-1, cudaSuccess) == cudaSuccess || run(PerDeviceOnce::kMaxDevices, cudaSuccess) == cudaSuccess)
        return fail(KXC_B200_ERR_INVALID, "per-device once: an ordinal out of range was accepted");
    return KXC_B200_OK;
}

extern "C" int32_t kxc_b200_nn_conv2d(void** packed_args, const kxc_b200_conv2d_desc* desc, void* stream) {
    KXC_TRY(require_device());
    ConvDims d;
    KXC_TRY(make_conv_dims(desc, "nn_conv2d", &d));
    if (!packed_args) return fail(KXC_B200_ERR_INVALID, "nn_conv2d: null packed_args");
    int i = 0;
    const float* data = static_cast<const float*>(packed_args[i++]);
    const float* weight = static_cast<const float*>(packed_args[i++]);
    const float* bias = (desc->flags & KXC_B200_BIAS) ? static_cast<const float*>(packed_args[i++]) : nullptr;
    const float* residual = (desc->flags & KXC_B200_RESIDUAL) ? static_cast<const float*>(packed_args[i++]) : nullptr;
    float* out = static_cast<float*>(packed_args[i++]);
    if (d.N == 0) return KXC_B200_OK;
    if (!data || !weight || !out || ((desc->flags & KXC_B200_BIAS) && !bias) || ((desc->flags & KXC_B200_RESIDUAL) && !residual))
        return fail(KXC_B200_ERR_INVALID, "nn_conv2d: null tensor pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int relu = (desc->flags & KXC_B200_RELU) ? 1 : 0;
    switch (desc->precision) {
        case KXC_B200_PREC_FP32:
            return conv2d_fp32_exact(data, weight, bias, residual, out, d, relu, s);
        case KXC_B200_PREC_TF32:
        case KXC_B200_PREC_BF16:
        case KXC_B200_PREC_TF32X3:
            return conv2d_tensor_core(data, weight, bias, residual, out, d, relu, desc->precision, s);
        default:
            return fail(KXC_B200_ERR_INVALID, "nn_conv2d: unknown precision %d", desc->precision);
    }
}

extern "C" int32_t kxc_b200_nn_conv2d_s8(void** packed_args, const kxc_b200_conv2d_desc* desc, void* stream) {
    KXC_TRY(require_device());
    ConvDims d;
    KXC_TRY(make_conv_dims(desc, "nn_conv2d_s8", &d));
    if (!packed_args) return fail(KXC_B200_ERR_INVALID, "nn_conv2d_s8: null packed_args");
    if (!(desc->flags & KXC_B200_BIAS) || (desc->flags & KXC_B200_RESIDUAL))
        return fail(KXC_B200_ERR_INVALID, "nn_conv2d_s8: flags must include BIAS and exclude RESIDUAL");
    if (d.N == 0) return KXC_B200_OK;
    for (int i = 0; i < 6; ++i)
        if (!packed_args[i]) return fail(KXC_B200_ERR_INVALID, "nn_conv2d_s8: null tensor pointer (arg %d)", i);
    return conv2d_s8_dispatch(static_cast<const int8_t*>(packed_args[0]), static_cast<const int8_t*>(packed_args[1]),
                              static_cast<const int32_t*>(packed_args[2]), static_cast<const int32_t*>(packed_args[3]),
                              static_cast<const int32_t*>(packed_args[4]), static_cast<int8_t*>(packed_args[5]), d,
                              (desc->flags & KXC_B200_RELU) ? 1 : 0, desc->precision == KXC_B200_PREC_SIMT ? 1 : 0,
                              (desc->flags & KXC_B200_NHWC) ? 1 : 0, static_cast<cudaStream_t>(stream));
}

extern "C" int32_t kxc_b200_nn_gemm(void** packed_args, const kxc_b200_gemm_desc* desc, void* stream) {
    KXC_TRY(require_device());
    if (!packed_args || !desc) return fail(KXC_B200_ERR_INVALID, "nn_gemm: bad arguments");
    if (desc->m < 0 || desc->n <= 0 || desc->k <= 0) return fail(KXC_B200_ERR_INVALID, "nn_gemm: bad shape");
    if (desc->transA != 0) return fail(KXC_B200_ERR_UNSUPPORTED, "nn_gemm currently does not support transA=1");
    int i = 0;
    const float* a = static_cast<const float*>(packed_args[i++]);
    const float* b = static_cast<const float*>(packed_args[i++]);
    const float* c = desc->has_c ? static_cast<const float*>(packed_args[i++]) : nullptr;
    float* out = static_cast<float*>(packed_args[i++]);
    if (desc->m == 0) return KXC_B200_OK;
    if (!a || !b || !out || (desc->has_c && !c)) return fail(KXC_B200_ERR_INVALID, "nn_gemm: null tensor pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    kxc_b200_gemm_desc g = *desc;
    if (!g.has_c) g.transB = 1;  // nn_dense: the weight is always [N, K]
    switch (g.precision) {
        case KXC_B200_PREC_FP32:
            return gemm_fp32_exact(a, b, c, out, g, s);
        case KXC_B200_PREC_TF32:
        case KXC_B200_PREC_BF16:
        case KXC_B200_PREC_TF32X3:
            return gemm_tensor_core(a, b, c, out, g, s);
        default:
            return fail(KXC_B200_ERR_INVALID, "nn_gemm: unknown precision %d", g.precision);
    }
}

extern "C" int32_t kxc_b200_matmul(void** packed_args, int32_t m, int32_t n, int32_t k, int32_t precision, void* stream) {
    KXC_TRY(require_device());
    if (!packed_args) return fail(KXC_B200_ERR_INVALID, "matmul: bad arguments");
    if (m < 0 || n < 0 || k <= 0) return fail(KXC_B200_ERR_INVALID, "matmul: bad shape");
    if (m == 0 || n == 0) return KXC_B200_OK;
    const float* a = static_cast<const float*>(packed_args[0]);
    const float* b = static_cast<const float*>(packed_args[1]);
    float* out = static_cast<float*>(packed_args[2]);
    if (!a || !b || !out) return fail(KXC_B200_ERR_INVALID, "matmul: null tensor pointer");
    // b is [K, N] and nothing is added: the internal form of that is "no C, transB = 0"
    const kxc_b200_gemm_desc g{m, n, k, 1.0f, 1.0f, 0, 0, 0, precision};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (precision) {
        case KXC_B200_PREC_FP32:
            return gemm_fp32_exact(a, b, nullptr, out, g, s);
        case KXC_B200_PREC_TF32:
        case KXC_B200_PREC_BF16:
        case KXC_B200_PREC_TF32X3:
            return gemm_tensor_core(a, b, nullptr, out, g, s);
        default:
            return fail(KXC_B200_ERR_INVALID, "matmul: unknown precision %d", precision);
    }
}

// kxc_b200_nn_conv2d_static_scratch: the tensor-core nn_conv2d for callers that must not allocate.
//
// The regular entry point converts its operands (NCHW fp32 -> channel-innermost bf16/tf32, OIHW ->
// packed weights) into a workspace it takes from the stream-ordered allocator on every call. Some
// hosts cannot do that: a runtime that has handed all device memory to its own pool and forbids the
// CUDA allocator afterwards, a real-time loop that may not take the allocator's locks, or code that
// runs while allocation is disallowed. For them the workspace here is a fixed array that is part of
// the library image: every GPU that loads libkxc_b200.so holds KXC_B200_STATIC_SCRATCH_BYTES of
// device memory for it until the process exits, whether or not this entry point is ever called.
//
// Rules that follow from sharing one array:
//  * the operands of one call must fit (converted activations + packed weights <= the array size);
//    larger problems are rejected with KXC_B200_ERR_NOMEM and a message naming both sizes;
//  * the array keeps the previous call's contents; every byte a call reads is first rewritten by
//    that call's own conversion kernels (padding channels included), so nothing needs clearing between
//    calls. The wait-status word of these kernels is a second static device word; it is only ever set on
//    failure, and kxc_b200_device_status reads and clears it together with the regular one;
//  * two calls whose GPU work overlaps (different streams, or different host threads on different
//    streams) race on the array. Issue them on one stream, or serialise them yourself;
//  * the first call on each device looks up the array's device address (cudaGetSymbolAddress, with
//    that device current). Make that first call outside any stream capture.
// The entry point calls no cudaMalloc / cudaFree / cudaMallocAsync and no allocating library routine.
#include "common.cuh"
#include "conv_common.cuh"
#include "conv_tc.cuh"
#include "layout.cuh"

#include <mutex>

#define KXC_B200_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)

namespace {

// In host code these names are host-side stand-ins for the device symbols, NOT device addresses: the
// addresses handed to kernels come from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[KXC_B200_STATIC_SCRATCH_BYTES];
static __device__ int g_static_status;

struct DeviceScratch {
    unsigned char* base = nullptr;
    int* status = nullptr;
    bool ready = false;
};

constexpr int kMaxDevices = 64;
DeviceScratch g_per_device[kMaxDevices];
std::mutex g_setup_mutex;

// Once per device, with that device current.
int32_t scratch_for_current_device(DeviceScratch* out) {
    int dev = 0;
    KXC_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return kxc_b200::fail(KXC_B200_ERR_INVALID, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    DeviceScratch& d = g_per_device[dev];
    if (!d.ready) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess)
            return kxc_b200::fail(KXC_B200_ERR_CUDA, "cudaGetSymbolAddress(static scratch) on device %d: %s", dev, cudaGetErrorString(e));
        d.base = static_cast<unsigned char*>(p);
        e = cudaGetSymbolAddress(&p, g_static_status);
        if (e != cudaSuccess)
            return kxc_b200::fail(KXC_B200_ERR_CUDA, "cudaGetSymbolAddress(static status) on device %d: %s", dev, cudaGetErrorString(e));
        d.status = static_cast<int*>(p);
        d.ready = true;
    }
    *out = d;
    return KXC_B200_OK;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

namespace kxc_b200 {
// The wait-status word of the static-scratch kernels on the current device, or nullptr while no call has resolved
// the symbols on that device (then no such kernel has run there and the word is still zero). Never allocates.
int32_t static_scratch_status_word(int** out) {
    int dev = 0;
    KXC_CUDA_TRY(cudaGetDevice(&dev));
    *out = nullptr;
    if (dev < 0 || dev >= kMaxDevices) return KXC_B200_OK;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_per_device[dev].ready) *out = g_per_device[dev].status;
    return KXC_B200_OK;
}
}  // namespace kxc_b200

using namespace kxc_b200;

extern "C" int64_t kxc_b200_static_scratch_bytes(void) { return (int64_t)KXC_B200_STATIC_SCRATCH_BYTES; }

extern "C" int32_t kxc_b200_nn_conv2d_static_scratch(void** packed_args, const kxc_b200_conv2d_desc* desc, void* stream) {
    KXC_TRY(require_device());
    if (!desc) return fail(KXC_B200_ERR_INVALID, "nn_conv2d_static_scratch: null descriptor");
    if (desc->n < 0 || desc->c <= 0 || desc->h <= 0 || desc->w <= 0 || desc->o <= 0 || desc->kh <= 0 || desc->kw <= 0 ||
        desc->stride_h <= 0 || desc->stride_w <= 0 || desc->pad_h < 0 || desc->pad_w < 0 || desc->dilation_h <= 0 || desc->dilation_w <= 0)
        return fail(KXC_B200_ERR_INVALID, "nn_conv2d_static_scratch: bad shape/stride/padding/dilation");
    const int64_t OH = conv_out_dim(desc->h, desc->kh, desc->stride_h, desc->pad_h, desc->dilation_h);
    const int64_t OW = conv_out_dim(desc->w, desc->kw, desc->stride_w, desc->pad_w, desc->dilation_w);
    if (OH <= 0 || OW <= 0) return fail(KXC_B200_ERR_INVALID, "nn_conv2d_static_scratch: empty output");
    const ConvDims d{desc->n, desc->c, desc->h, desc->w, desc->o, desc->kh, desc->kw, desc->stride_h, desc->stride_w,
                     desc->pad_h, desc->pad_w, desc->dilation_h, desc->dilation_w, (int)OH, (int)OW};
    if (!packed_args) return fail(KXC_B200_ERR_INVALID, "nn_conv2d_static_scratch: null packed_args");
    int i = 0;
    const float* data = static_cast<const float*>(packed_args[i++]);
    const float* weight = static_cast<const float*>(packed_args[i++]);
    const float* bias = (desc->flags & KXC_B200_BIAS) ? static_cast<const float*>(packed_args[i++]) : nullptr;
    const float* residual = (desc->flags & KXC_B200_RESIDUAL) ? static_cast<const float*>(packed_args[i++]) : nullptr;
    float* out = static_cast<float*>(packed_args[i++]);
    if (d.N == 0) return KXC_B200_OK;
    if (!data || !weight || !out || ((desc->flags & KXC_B200_BIAS) && !bias) || ((desc->flags & KXC_B200_RESIDUAL) && !residual))
        return fail(KXC_B200_ERR_INVALID, "nn_conv2d_static_scratch: null tensor pointer");
    if (desc->precision != KXC_B200_PREC_BF16 && desc->precision != KXC_B200_PREC_TF32)
        return fail(KXC_B200_ERR_INVALID, "nn_conv2d_static_scratch: precision must be KXC_B200_PREC_BF16 or KXC_B200_PREC_TF32 "
                                          "(the fp32 mode of kxc_b200_nn_conv2d needs no workspace)");
    if (!(d.SH == d.SW && (d.SH == 1 || d.SH == 2) && !(d.SH == 2 && (d.H < 2 || d.W < 2)) && d.N <= 65535))
        return fail(KXC_B200_ERR_UNSUPPORTED, "nn_conv2d_static_scratch: the tensor-core path needs equal strides of 1 or 2");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int relu = (desc->flags & KXC_B200_RELU) ? 1 : 0;

    const TcDType dt = desc->precision == KXC_B200_PREC_BF16 ? kTcBF16 : kTcTF32;
    const int eb = tc_elem_bytes(dt);
    const int cpad = tc_channel_pad(dt, d.C);
    const size_t act_bytes = align_up((size_t)d.N * d.H * d.W * cpad * eb, 1024);
    const size_t w_bytes = align_up((size_t)d.O * d.KH * d.KW * cpad * eb, 1024);
    if (act_bytes + w_bytes > (size_t)KXC_B200_STATIC_SCRATCH_BYTES)
        return fail(KXC_B200_ERR_NOMEM,
                    "nn_conv2d_static_scratch: this convolution needs %zu bytes of workspace, the static scratch holds %u; "
                    "use kxc_b200_nn_conv2d or a smaller batch",
                    act_bytes + w_bytes, KXC_B200_STATIC_SCRATCH_BYTES);
    DeviceScratch sc;
    KXC_TRY(scratch_for_current_device(&sc));
    unsigned char* act = sc.base;
    unsigned char* wp = sc.base + act_bytes;
    KXC_TRY(nchw_to_nhwc(data, act, dt, d.N, d.C, d.H * d.W, cpad, s));
    KXC_TRY(pack_weights_ohwi(weight, wp, dt, d.O, d.C, d.KH, d.KW, cpad, s));
    TcParams p{};
    TcConfig cfg{};
    KXC_TRY(tc_setup_conv(&p, &cfg, dt, kOutNCHW_F32, act, wp, d.N, d.H, d.W, cpad, d.O, d.KH, d.KW, d.SH, d.PH, d.PW, d.DH, d.DW,
                          sc.status));
    p.bias = bias;
    p.residual = residual;
    p.out = out;
    p.relu = relu;
    tc_finish_params(&p);
    return tc_launch(cfg, p, s);
}

// Per-operator glue between the reference-layout entry points (NCHW fp32 / int8 tensors) and the
// tensor-core implicit-GEMM kernel: operand conversion into a stream-ordered workspace, parameter
// set-up, launch. Shapes the tensor-core path does not take fall back to the CUDA-core kernels
// (still on the GPU; there is no CPU path).
#include "common.cuh"
#include "conv_common.cuh"
#include "conv_tc.cuh"
#include "layout.cuh"
#include "sm100.cuh"
#include "conv_rowstack.cuh"
#include "conv_stem.cuh"

#include <mutex>

namespace kxc_b200 {

namespace {

// The library's own stream-ordered memory pool, one per device, that keeps what it has allocated (release threshold =
// unlimited). The device's default pool gives freed memory back to the driver at the next synchronisation, so a caller that
// synchronises between calls would pay a fresh device allocation (milliseconds for tens of MB) inside every call.
int32_t scratch_pool(cudaMemPool_t* out) {
    static std::mutex mu;
    static cudaMemPool_t pools[PerDeviceOnce::kMaxDevices] = {};
    int dev = 0;
    KXC_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= PerDeviceOnce::kMaxDevices) return fail(KXC_B200_ERR_INVALID, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (pools[dev] == nullptr) {
        cudaMemPoolProps props = {};
        props.allocType = cudaMemAllocationTypePinned;
        props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice;
        props.location.id = dev;
        cudaMemPool_t pool = nullptr;
        KXC_CUDA_TRY(cudaMemPoolCreate(&pool, &props));
        uint64_t keep = UINT64_MAX;
        KXC_CUDA_TRY(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
        pools[dev] = pool;
    }
    *out = pools[dev];
    return KXC_B200_OK;
}

// Stream-ordered scratch: allocated and freed on the caller's stream, so the call stays asynchronous.
struct StreamScratch {
    void* ptr = nullptr;
    cudaStream_t stream;
    explicit StreamScratch(cudaStream_t s) : stream(s) {}
    int32_t alloc(size_t bytes) {
        cudaMemPool_t pool = nullptr;
        KXC_TRY(scratch_pool(&pool));
        cudaError_t e = cudaMallocFromPoolAsync(&ptr, bytes, pool, stream);
        if (e != cudaSuccess) {
            ptr = nullptr;
            return fail(KXC_B200_ERR_NOMEM, "workspace of %zu bytes: %s", bytes, cudaGetErrorString(e));
        }
        return KXC_B200_OK;
    }
    ~StreamScratch() {
        if (ptr) cudaFreeAsync(ptr, stream);
    }
};

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

bool tc_shape_ok(const ConvDims& d) {
    return d.SH == d.SW && (d.SH == 1 || d.SH == 2) && !(d.SH == 2 && (d.H < 2 || d.W < 2)) && d.N <= 65535;
}

}  // namespace

int32_t conv2d_tensor_core(const float* data, const float* weight, const float* bias, const float* residual, float* out,
                           const ConvDims& d, int relu, int precision, cudaStream_t s) {
    if (!tc_shape_ok(d)) return conv2d_fp32_exact(data, weight, bias, residual, out, d, relu, s);
    if (precision == KXC_B200_PREC_TF32X3) {
        // Three tf32 passes into the same fp32 output, small terms first: x_lo*w_hi (+ the caller's residual), then
        // x_hi*w_lo + that, then x_hi*w_hi + bias + that, ReLU last. Each pass reads the previous sum through the
        // epilogue's residual input; reading and writing the same element from the same thread is safe in place.
        const int cpad = tc_channel_pad(kTcTF32, d.C);
        const size_t act_bytes = align_up((size_t)d.N * d.H * d.W * cpad * 4, 1024);
        const size_t w_bytes = align_up((size_t)d.O * d.KH * d.KW * cpad * 4, 1024);
        StreamScratch ws(s);
        KXC_TRY(ws.alloc(2 * act_bytes + 2 * w_bytes));
        uint8_t* act_hi = static_cast<uint8_t*>(ws.ptr);
        uint8_t* act_lo = act_hi + act_bytes;
        uint8_t* w_hi = act_lo + act_bytes;
        uint8_t* w_lo = w_hi + w_bytes;
        KXC_TRY(nchw_to_nhwc(data, act_hi, kTcTF32, d.N, d.C, d.H * d.W, cpad, s));
        KXC_TRY(nchw_to_nhwc(data, act_lo, kTcTF32, d.N, d.C, d.H * d.W, cpad, s, true));
        KXC_TRY(pack_weights_ohwi(weight, w_hi, kTcTF32, d.O, d.C, d.KH, d.KW, cpad, s));
        KXC_TRY(pack_weights_ohwi(weight, w_lo, kTcTF32, d.O, d.C, d.KH, d.KW, cpad, s, true));
        const uint8_t* as[3] = {act_lo, act_hi, act_hi};
        const uint8_t* wsrc[3] = {w_hi, w_lo, w_hi};
        for (int pass = 0; pass < 3; ++pass) {
            TcParams p{};
            TcConfig cfg{};
            KXC_TRY(tc_setup_conv(&p, &cfg, kTcTF32, kOutNCHW_F32, as[pass], wsrc[pass], d.N, d.H, d.W, cpad, d.O, d.KH, d.KW, d.SH,
                                  d.PH, d.PW, d.DH, d.DW));
            p.bias = pass == 2 ? bias : nullptr;
            p.residual = pass == 0 ? residual : out;
            p.out = out;
            p.relu = pass == 2 ? relu : 0;
            tc_finish_params(&p);
            KXC_TRY(tc_launch(cfg, p, s));
        }
        return KXC_B200_OK;
    }
    const TcDType dt = precision == KXC_B200_PREC_BF16 ? kTcBF16 : kTcTF32;
    const int eb = tc_elem_bytes(dt);
    const int cpad = tc_channel_pad(dt, d.C);
    const size_t act_bytes = align_up((size_t)d.N * d.H * d.W * cpad * eb, 1024);
    const size_t w_bytes = align_up((size_t)d.O * d.KH * d.KW * cpad * eb, 1024);
    StreamScratch ws(s);
    KXC_TRY(ws.alloc(act_bytes + w_bytes));
    uint8_t* act = static_cast<uint8_t*>(ws.ptr);
    uint8_t* wp = act + act_bytes;
    KXC_TRY(nchw_to_nhwc(data, act, dt, d.N, d.C, d.H * d.W, cpad, s));
    KXC_TRY(pack_weights_ohwi(weight, wp, dt, d.O, d.C, d.KH, d.KW, cpad, s));
    TcParams p{};
    TcConfig cfg{};
    KXC_TRY(tc_setup_conv(&p, &cfg, dt, kOutNCHW_F32, act, wp, d.N, d.H, d.W, cpad, d.O, d.KH, d.KW, d.SH, d.PH, d.PW, d.DH,
                          d.DW));
    p.bias = bias;
    p.residual = residual;
    p.out = out;
    p.relu = relu;
    tc_finish_params(&p);
    return tc_launch(cfg, p, s);
}

int32_t conv2d_s8_dispatch(const int8_t* data, const int8_t* weight, const int32_t* bias, const int32_t* multiplier,
                           const int32_t* shift, int8_t* out, const ConvDims& d, int relu, int force_simt, int nhwc,
                           cudaStream_t s) {
    const TcDType dt = kTcS8;
    const int cpad = tc_channel_pad(dt, d.C);
    // few-channel stride-2 first layer (the 7x7 stem): pixels packed to 8 bytes, direct kernel, K = 7 x 64 bytes instead of
    // 49 taps x 32 padded channels. Both layouts of the entry point take it (NHWC: data [N,H,W,C], weight [O,KH,KW,C]).
    const int stem_hp = (d.H + 2 * d.PH + 1) & ~1;
    const int stem_wp = ((d.W + 2 * d.PW > 2 * (d.OW - 1) + 8 ? d.W + 2 * d.PW : 2 * (d.OW - 1) + 8) + 3) / 4 * 4;
    const bool stem_ok = !force_simt && tc_shape_ok(d) && d.SH == 2 && d.SW == 2 && d.DH == 1 && d.DW == 1 &&
                         stem_direct_s8_applicable(d.C, d.O, d.KH, d.KW, 2, 1, d.W, d.OW, stem_wp);
    // 64 -> 64 channels, 3x3, stride 1: the row-stacked kernel (one box load per tile instead of nine)
    static const bool rowstack_enabled = [] {
        const char* e = getenv("KXC_B200_ROWSTACK_S8");
        return !(e != nullptr && e[0] == '0');
    }();
    const bool rowstack_ok = rowstack_enabled && !force_simt && tc_shape_ok(d) &&
                             rowstack3x3_s8_applicable(d.C, d.O, d.KH, d.KW, d.SH == d.SW ? d.SH : 0, d.PH, d.PW, d.DH, d.DW);
    auto run_stem = [&](bool nhwc_layout) -> int32_t {
        const size_t x_bytes = align_up((size_t)d.N * stem_hp * stem_wp * 8, 1024);
        const size_t w_bytes = align_up(stem_direct_weight_bytes(d.KH), 1024);
        StreamScratch ws(s);
        KXC_TRY(ws.alloc(x_bytes + w_bytes));
        uint8_t* px = static_cast<uint8_t*>(ws.ptr);
        uint8_t* pw = px + x_bytes;
        KXC_TRY(stem_direct_s8_pack(data, weight, px, pw, d.N, d.C, d.H, d.W, d.O, d.KH, d.KW, stem_hp, stem_wp, d.PH, d.PW, nhwc_layout, s));
        TcParams p{};
        KXC_TRY(stem_direct_setup(&p, px, pw, d.N, d.OH, d.OW, d.KH, stem_hp, stem_wp));
        p.bias_i32 = bias;
        p.multiplier = multiplier;
        p.shift = shift;
        p.out = out;
        p.relu = relu;
        tc_finish_params(&p);
        return stem_direct_s8_launch(p, nhwc_layout, s);
    };
    if (nhwc) {
        // operands already NHWC / OHWI with the kernel's channel granularity: straight to the tensor-core kernel
        if (force_simt || !tc_shape_ok(d)) return fail(KXC_B200_ERR_UNSUPPORTED, "nn_conv2d_s8: the NHWC form exists for the tensor-core path only");
        if (stem_ok && d.C <= 8 && aligned16(out)) return run_stem(true);
        if (cpad != d.C || (d.O & 15) != 0 || !aligned16(data) || !aligned16(weight) || !aligned16(out))
            return fail(KXC_B200_ERR_INVALID, "nn_conv2d_s8: NHWC operands need C = 32/64/128k channels, O a multiple of 16 and 16-byte aligned pointers");
        TcParams p{};
        if (rowstack_ok) {
            KXC_TRY(rowstack3x3_s8_setup(&p, data, weight, d.N, d.H, d.W));
            p.bias_i32 = bias;
            p.multiplier = multiplier;
            p.shift = shift;
            p.out = out;
            p.relu = relu;
            tc_finish_params(&p);
            return rowstack3x3_s8_launch(p, s);
        }
        TcConfig cfg{};
        KXC_TRY(tc_setup_conv(&p, &cfg, dt, kOutNHWC_S8, data, weight, d.N, d.H, d.W, cpad, d.O, d.KH, d.KW, d.SH, d.PH, d.PW, d.DH,
                              d.DW));
        p.bias_i32 = bias;
        p.multiplier = multiplier;
        p.shift = shift;
        p.out = out;
        p.relu = relu;
        tc_finish_params(&p);
        return tc_launch(cfg, p, s);
    }
    if (force_simt || !tc_shape_ok(d)) return conv2d_s8_exact(data, weight, bias, multiplier, shift, out, d, relu, s);
    if (stem_ok) return run_stem(false);
    // A 1x1 convolution of stride > 1 without padding reads one pixel in stride^2: only those are converted, and the
    // kernel runs as a stride-1 convolution over the subsampled tensor (a quarter of the conversion and of the kernel's
    // loads for the downsample branches of a ResNet).
    const bool subsample = d.KH == 1 && d.KW == 1 && d.PH == 0 && d.PW == 0 && d.SH == d.SW && d.SH > 1 && (cpad & 3) == 0 &&
                           d.N <= 65535;
    const int in_h = d.H, in_w = d.W;
    const int conv_h = subsample ? d.OH : d.H, conv_w = subsample ? d.OW : d.W;  // the tensor the kernel convolves
    const size_t act_bytes = align_up((size_t)d.N * conv_h * conv_w * cpad, 1024);
    const size_t w_bytes = align_up((size_t)d.O * d.KH * d.KW * cpad, 1024);
    // Result layout. A thread of the epilogue owns one pixel, so its NCHW stores are single bytes whose neighbours in
    // memory belong to the next pixel of the same tile row: runs of BW bytes. With the narrow tiles of the deep layers
    // (BW <= 2) that costs more than the kernel itself (512 -> 512 channels at 7x7, 256 images: 100 us against 35 us for
    // the NHWC form), so those layers store NHWC into the workspace and a byte transpose writes the reference layout.
    int bw = 0, bh = 0, bni = 0;
    tc_pick_tile(d.N, d.OH, d.OW, &bw, &bh, &bni);
    const bool two_step = (bw <= 2 && (d.O & 15) == 0) || rowstack_ok;  // (the row-stacked kernel writes NHWC only)
    const size_t out_bytes = two_step ? align_up((size_t)d.N * d.OH * d.OW * d.O, 1024) : 0;
    StreamScratch ws(s);
    KXC_TRY(ws.alloc(act_bytes + w_bytes + out_bytes));
    uint8_t* act = static_cast<uint8_t*>(ws.ptr);
    uint8_t* wp = act + act_bytes;
    int8_t* out_nhwc = reinterpret_cast<int8_t*>(wp + w_bytes);
    if (subsample) {
        KXC_TRY(nchw_to_nhwc_s8_subsample(data, reinterpret_cast<int8_t*>(act), d.N, d.C, in_h, in_w, d.OH, d.OW, d.SH, cpad, s));
    } else {
        KXC_TRY(nchw_to_nhwc(data, act, dt, d.N, d.C, d.H * d.W, cpad, s));
    }
    KXC_TRY(pack_weights_ohwi(weight, wp, dt, d.O, d.C, d.KH, d.KW, cpad, s));
    TcParams p{};
    TcConfig cfg{};
    if (rowstack_ok) {
        KXC_TRY(rowstack3x3_s8_setup(&p, act, wp, d.N, d.H, d.W));
    } else {
        KXC_TRY(tc_setup_conv(&p, &cfg, dt, two_step ? kOutNHWC_S8 : kOutNCHW_S8, act, wp, d.N, conv_h, conv_w, cpad, d.O, d.KH, d.KW,
                              subsample ? 1 : d.SH, d.PH, d.PW, d.DH, d.DW));
    }
    p.bias_i32 = bias;
    p.multiplier = multiplier;
    p.shift = shift;
    p.out = two_step ? out_nhwc : out;
    p.relu = relu;
    tc_finish_params(&p);
    if (rowstack_ok) {
        KXC_TRY(rowstack3x3_s8_launch(p, s));
    } else {
        KXC_TRY(tc_launch(cfg, p, s));
    }
    if (two_step) return nhwc_to_nchw_s8(out_nhwc, out, d.N, d.O, d.OH * d.OW, s);
    return KXC_B200_OK;
}

int32_t gemm_tensor_core(const float* a, const float* b, const float* c, float* out, const kxc_b200_gemm_desc& g,
                         cudaStream_t s) {
    // alpha/beta scaling is a separately rounded multiply in the reference; only the common
    // alpha = beta = 1 form is fused into the tensor-core epilogue.
    if ((g.has_c && ((double)g.alpha != 1.0 || (double)g.beta != 1.0)) || g.m > 65535 * 128)
        return gemm_fp32_exact(a, b, c, out, g, s);
    if (g.precision == KXC_B200_PREC_TF32X3) {
        // as in conv2d_tensor_core: a_lo*b_hi, + a_hi*b_lo, + a_hi*b_hi + c
        const int kpad = tc_channel_pad(kTcTF32, g.k);
        const size_t a_bytes = align_up((size_t)g.m * kpad * 4, 1024);
        const size_t b_bytes = align_up((size_t)g.n * kpad * 4, 1024);
        StreamScratch ws(s);
        KXC_TRY(ws.alloc(2 * a_bytes + 2 * b_bytes));
        uint8_t* part[4];  // a_hi, a_lo, b_hi, b_lo
        part[0] = static_cast<uint8_t*>(ws.ptr);
        part[1] = part[0] + a_bytes;
        part[2] = part[1] + a_bytes;
        part[3] = part[2] + b_bytes;
        for (int lo = 0; lo < 2; ++lo) {
            KXC_TRY(convert_rows(a, part[lo], kTcTF32, g.m, g.k, kpad, s, lo == 1));
            if (g.transB)
                KXC_TRY(convert_rows(b, part[2 + lo], kTcTF32, g.n, g.k, kpad, s, lo == 1));
            else
                KXC_TRY(nchw_to_nhwc(b, part[2 + lo], kTcTF32, 1, g.k, g.n, kpad, s, lo == 1));
        }
        const uint8_t* as[3] = {part[1], part[0], part[0]};
        const uint8_t* bs[3] = {part[2], part[3], part[2]};
        for (int pass = 0; pass < 3; ++pass) {
            TcParams p{};
            TcConfig cfg{};
            KXC_TRY(tc_setup_conv(&p, &cfg, kTcTF32, kOutNHWC_F32, as[pass], bs[pass], g.m, 1, 1, kpad, g.n, 1, 1, 1, 0, 0, 1, 1));
            p.bias = (pass == 2 && g.has_c) ? c : nullptr;
            p.residual = pass == 0 ? nullptr : out;
            p.out = out;
            p.relu = 0;
            tc_finish_params(&p);
            KXC_TRY(tc_launch(cfg, p, s));
        }
        return KXC_B200_OK;
    }
    const TcDType dt = g.precision == KXC_B200_PREC_BF16 ? kTcBF16 : kTcTF32;
    const int eb = tc_elem_bytes(dt);
    const int kpad = tc_channel_pad(dt, g.k);
    const size_t a_bytes = align_up((size_t)g.m * kpad * eb, 1024);
    const size_t b_bytes = align_up((size_t)g.n * kpad * eb, 1024);
    StreamScratch ws(s);
    KXC_TRY(ws.alloc(a_bytes + b_bytes));
    uint8_t* ap = static_cast<uint8_t*>(ws.ptr);
    uint8_t* bp = ap + a_bytes;
    KXC_TRY(convert_rows(a, ap, dt, g.m, g.k, kpad, s));
    if (g.transB) {
        KXC_TRY(convert_rows(b, bp, dt, g.n, g.k, kpad, s));  // b is [N, K]
    } else {
        KXC_TRY(nchw_to_nhwc(b, bp, dt, 1, g.k, g.n, kpad, s));  // b is [K, N] -> [N, Kpad]
    }
    TcParams p{};
    TcConfig cfg{};
    // A dense layer is a 1x1 convolution over an M x 1 x 1 "image" batch.
    KXC_TRY(tc_setup_conv(&p, &cfg, dt, kOutNHWC_F32, ap, bp, g.m, 1, 1, kpad, g.n, 1, 1, 1, 0, 0, 1, 1));
    p.bias = g.has_c ? c : nullptr;
    p.out = out;
    p.relu = 0;
    tc_finish_params(&p);
    return tc_launch(cfg, p, s);
}

}  // namespace kxc_b200

using namespace kxc_b200;

// Reads (and clears) the device status words written by a tensor-core kernel whose bounded wait ran
// out: the regular one and the one of the static-scratch entry point. Synchronises the stream.
// 0 = every kernel so far completed its protocol. Allocates nothing once the regular word exists.
extern "C" int32_t kxc_b200_device_status(void* stream, int32_t* status_out) {
    KXC_TRY(require_device());
    int* words[2] = {nullptr, nullptr};
    KXC_TRY(tc_status_word(&words[0]));
    KXC_TRY(static_scratch_status_word(&words[1]));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int host[2] = {0, 0};
    for (int i = 0; i < 2; ++i)
        if (words[i]) KXC_CUDA_TRY(cudaMemcpyAsync(&host[i], words[i], sizeof(int), cudaMemcpyDeviceToHost, s));
    KXC_CUDA_TRY(cudaStreamSynchronize(s));
    for (int i = 0; i < 2; ++i)
        if (host[i] != 0) KXC_CUDA_TRY(cudaMemsetAsync(words[i], 0, sizeof(int), s));
    const int combined = host[0] | host[1];
    if (status_out) *status_out = combined;
    if (combined != 0)
        return fail(KXC_B200_ERR_DEVICE_WAIT, "a tensor-core kernel gave up a bounded wait (status %d%s)", combined,
                    host[1] != 0 ? ", static-scratch entry point" : "");
    return KXC_B200_OK;
}

// ---- self tests -----------------------------------------------------------------------------------------
namespace kxc_b200 {
namespace {
// One CTA waits, through the same bounded wait every tensor-core kernel uses, on an mbarrier that nothing ever
// arrives on. After `limit_ns` the wait gives up, the kernel reports into the status word and returns normally.
__global__ void bounded_wait_selftest_kernel(uint64_t limit_ns, int* status, int* gave_up) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        sm100::mbar_init(sm100::smem_u32(&bar), 1);
        sm100::mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const bool arrived = sm100::mbar_wait_bounded(sm100::smem_u32(&bar), 0, &abort_flag, limit_ns);
        *gave_up = arrived ? 0 : 1;
        if (!arrived) atomicExch(status, KXC_B200_ERR_DEVICE_WAIT);
    }
}
}  // namespace
}  // namespace kxc_b200

extern "C" int32_t kxc_b200_selftest_bounded_wait(int64_t limit_ns, void* stream, int32_t* gave_up_out) {
    KXC_TRY(require_device());
    if (limit_ns <= 0 || limit_ns > 100000000ll) return fail(KXC_B200_ERR_INVALID, "selftest_bounded_wait: limit must be in (0, 100 ms]");
    int* word = nullptr;
    KXC_TRY(tc_status_word(&word));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int* flag = nullptr;
    KXC_CUDA_TRY(cudaMallocAsync(&flag, sizeof(int), s));
    KXC_CUDA_TRY(cudaMemsetAsync(flag, 0, sizeof(int), s));
    bounded_wait_selftest_kernel<<<1, 32, 0, s>>>((uint64_t)limit_ns, word, flag);
    const int32_t rc = check_launch("bounded_wait_selftest_kernel");
    int host = 0;
    cudaError_t e = cudaMemcpyAsync(&host, flag, sizeof(int), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    cudaFreeAsync(flag, s);
    if (rc != KXC_B200_OK) return rc;
    if (e != cudaSuccess) return fail(KXC_B200_ERR_CUDA, "selftest_bounded_wait: %s", cudaGetErrorString(e));
    if (gave_up_out) *gave_up_out = host;
    return KXC_B200_OK;
}

// CUDA-core (SIMT) contraction kernels in the reference's own operation order.
//
// These are the KXC_B200_PREC_FP32 mode of nn_conv2d / nn_gemm and the integer-exact form of the
// int8 convolution. Each output element is one thread's sequential reduction
//   acc = 0; for rc, rh, rw: acc = acc + (inb ? x : 0) * w          include/te/topi/nn.h:107-158
// with separately rounded multiply and add (__fmul_rn/__fadd_rn are never contracted into FMA), so
// fp32 results are bit-identical to the reference's CPU lowering. They also serve shapes the
// tensor-core path does not take (dilation, channel counts that do not fill a K block).
#include "common.cuh"
#include "conv_common.cuh"

namespace kxc_b200 {
namespace {

constexpr int kThreads = 128;

template <typename TIn, typename TAcc>
__device__ __forceinline__ TAcc mac_exact(TAcc acc, TIn x, TIn w);
template <>
__device__ __forceinline__ float mac_exact<float, float>(float acc, float x, float w) {
    return __fadd_rn(acc, __fmul_rn(x, w));
}
template <>
__device__ __forceinline__ int32_t mac_exact<int8_t, int32_t>(int32_t acc, int8_t x, int8_t w) {
    return acc + (int32_t)x * (int32_t)w;
}

// One thread per output element, ow fastest so a warp reads contiguous input columns; the weight
// address is warp-uniform for most warps (broadcast load).
template <typename TIn, typename TAcc, typename Epilogue>
__global__ void __launch_bounds__(kThreads) conv2d_direct_kernel(const TIn* __restrict__ data,
                                                                 const TIn* __restrict__ weight, ConvDims d,
                                                                 Epilogue epi) {
    const int64_t total = (int64_t)d.N * d.O * d.OH * d.OW;
    for (int64_t lin = (int64_t)blockIdx.x * kThreads + threadIdx.x; lin < total; lin += (int64_t)gridDim.x * kThreads) {
        const int ow = (int)(lin % d.OW);
        int64_t t = lin / d.OW;
        const int oh = (int)(t % d.OH);
        t /= d.OH;
        const int o = (int)(t % d.O);
        const int n = (int)(t / d.O);
        const TIn* xn = data + (int64_t)n * d.C * d.H * d.W;
        const TIn* wo = weight + (int64_t)o * d.C * d.KH * d.KW;
        TAcc acc = 0;
        for (int rc = 0; rc < d.C; ++rc) {
            const TIn* xc = xn + (int64_t)rc * d.H * d.W;
            const TIn* wc = wo + rc * d.KH * d.KW;
            for (int rh = 0; rh < d.KH; ++rh) {
                const int ih = oh * d.SH + rh * d.DH - d.PH;
                const bool inb_h = (ih >= 0) && (ih < d.H);
                for (int rw = 0; rw < d.KW; ++rw) {
                    const int iw = ow * d.SW + rw * d.DW - d.PW;
                    const bool inb = inb_h && (iw >= 0) && (iw < d.W);
                    const TIn xv = inb ? __ldg(xc + (int64_t)ih * d.W + iw) : (TIn)0;
                    acc = mac_exact<TIn, TAcc>(acc, xv, __ldg(wc + rh * d.KW + rw));
                }
            }
        }
        epi(acc, lin, o);
    }
}

struct EpilogueF32 {
    const float* bias;
    const float* residual;
    float* out;
    int relu;
    __device__ __forceinline__ void operator()(float acc, int64_t lin, int o) const {
        float v = acc;
        if (bias) v = __fadd_rn(v, __ldg(bias + o));
        if (residual) v = __fadd_rn(v, __ldg(residual + lin));
        if (relu) v = v > 0.0f ? v : 0.0f;
        out[lin] = v;
    }
};

struct EpilogueS8 {
    const int32_t* bias;
    const int32_t* multiplier;
    const int32_t* shift;
    int8_t* out;
    int relu;
    __device__ __forceinline__ void operator()(int32_t acc, int64_t lin, int o) const {
        out[lin] = requantize_s8(acc + __ldg(bias + o), __ldg(multiplier + o), __ldg(shift + o), relu);
    }
};

// nn_dense / nn_gemm in reference order: acc = 0; acc += a[i,k]*b[j,k]; (*alpha); + (beta*)c[j]
// (include/te/topi/nn.h:48-101, src/relay/op/nn/dense.cc:34-61).
__global__ void __launch_bounds__(kThreads) gemm_direct_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                               const float* __restrict__ c, float* __restrict__ out,
                                                               int M, int N, int K, float alpha, float beta, int transB,
                                                               int has_c) {
    const int64_t total = (int64_t)M * N;
    for (int64_t lin = (int64_t)blockIdx.x * kThreads + threadIdx.x; lin < total; lin += (int64_t)gridDim.x * kThreads) {
        const int j = (int)(lin % N);
        const int i = (int)(lin / N);
        float acc = 0.0f;
        if (transB) {
            for (int k = 0; k < K; ++k) acc = __fadd_rn(acc, __fmul_rn(__ldg(a + (int64_t)i * K + k), __ldg(b + (int64_t)j * K + k)));
        } else {
            for (int k = 0; k < K; ++k) acc = __fadd_rn(acc, __fmul_rn(__ldg(a + (int64_t)i * K + k), __ldg(b + (int64_t)k * N + j)));
        }
        if (has_c) {
            if ((double)alpha != 1.0) acc = __fmul_rn(acc, alpha);
            float bias = __ldg(c + j);
            if ((double)beta != 1.0) bias = __fmul_rn(bias, beta);
            acc = __fadd_rn(acc, bias);
        }
        out[lin] = acc;
    }
}

int grid_for(int64_t items) {
    int64_t blocks = (items + kThreads - 1) / kThreads;
    const int64_t cap = (int64_t)kNumSMs * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

}  // namespace

int32_t conv2d_fp32_exact(const float* data, const float* weight, const float* bias, const float* residual, float* out,
                          const ConvDims& d, int relu, cudaStream_t s) {
    const int64_t total = (int64_t)d.N * d.O * d.OH * d.OW;
    if (total == 0) return KXC_B200_OK;
    EpilogueF32 epi{bias, residual, out, relu};
    conv2d_direct_kernel<float, float, EpilogueF32><<<grid_for(total), kThreads, 0, s>>>(data, weight, d, epi);
    return check_launch("nn_conv2d (fp32)");
}

int32_t conv2d_s8_exact(const int8_t* data, const int8_t* weight, const int32_t* bias, const int32_t* multiplier,
                        const int32_t* shift, int8_t* out, const ConvDims& d, int relu, cudaStream_t s) {
    const int64_t total = (int64_t)d.N * d.O * d.OH * d.OW;
    if (total == 0) return KXC_B200_OK;
    EpilogueS8 epi{bias, multiplier, shift, out, relu};
    conv2d_direct_kernel<int8_t, int32_t, EpilogueS8><<<grid_for(total), kThreads, 0, s>>>(data, weight, d, epi);
    return check_launch("nn_conv2d_s8 (direct)");
}

int32_t gemm_fp32_exact(const float* a, const float* b, const float* c, float* out, const kxc_b200_gemm_desc& g,
                        cudaStream_t s) {
    const int64_t total = (int64_t)g.m * g.n;
    if (total == 0) return KXC_B200_OK;
    gemm_direct_kernel<<<grid_for(total), kThreads, 0, s>>>(a, b, c, out, g.m, g.n, g.k, g.alpha, g.beta, g.transB, g.has_c);
    return check_launch("nn_gemm (fp32)");
}

}  // namespace kxc_b200

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

// Register-tiled fp32 form of the same reduction: a block of 128 threads computes 64 output channels x kPT * 2 * kOT
// consecutive output pixels (flattened over n, oh, ow), a thread kOT channels x kPT pixels. Every output element is still
// ONE sequential chain acc = acc + x * w over rc, rh, rw with separately rounded multiply and add, so the bits are those
// of the one-thread-per-output kernel above; only the number of loads per multiply changes (an input value serves kOT
// channels, a weight kPT pixels). Weights of `rc_block` input channels at a time are staged in shared memory as
// [rc][tap][64 channels], so a thread's weights are one or two 16-byte broadcast loads. kKW: the filter width at compile time (1, 3, 7) so that a filter row's loads are all
// issued before its arithmetic; 0 = any.
constexpr int kTileO = 64, kTileThreads = 128;

template <int kKW, int kOT, int kPT, typename Epilogue>
__global__ void __launch_bounds__(kTileThreads) conv2d_tiled_f32_kernel(const float* __restrict__ data, const float* __restrict__ weight,
                                                                        ConvDims d, int rc_block, Epilogue epi) {
    static_assert(kOT == 4 || kOT == 8, "one or two float4 of weights per thread");
    constexpr int kOG = kTileO / kOT;            // channel groups of a block
    constexpr int kPG = kTileThreads / kOG;      // pixel groups of a block
    constexpr int kTileP = kPG * kPT;
    extern __shared__ __align__(16) float w_s[];  // [rc_block][KH*KW][kTileO]
    const int KW = kKW > 0 ? kKW : d.KW;
    const int taps = d.KH * KW;
    const int plane_out = d.OH * d.OW;
    const int64_t P = (int64_t)d.N * plane_out;
    const int o0 = blockIdx.y * kTileO;
    const int64_t p0 = (int64_t)blockIdx.x * kTileP;
    const int pg = threadIdx.x % kPG;   // pixels p0 + pg + kPG e: consecutive lanes read consecutive pixels
    const int og = threadIdx.x / kPG;   // channels o0 + kOT og ..
    int ih0[kPT], iw0[kPT];
    bool pix_ok[kPT];
    const float* xn[kPT];
#pragma unroll
    for (int e = 0; e < kPT; ++e) {
        const int64_t p = p0 + pg + kPG * e;
        pix_ok[e] = p < P;
        const int n = pix_ok[e] ? (int)(p / plane_out) : 0;
        const int rem = pix_ok[e] ? (int)(p - (int64_t)n * plane_out) : 0;
        const int oh = rem / d.OW, ow = rem - oh * d.OW;
        ih0[e] = oh * d.SH - d.PH;
        iw0[e] = ow * d.SW - d.PW;
        xn[e] = data + (int64_t)n * d.C * d.H * d.W;
    }
    float acc[kOT][kPT];
#pragma unroll
    for (int j = 0; j < kOT; ++j)
#pragma unroll
        for (int e = 0; e < kPT; ++e) acc[j][e] = 0.0f;
    const int64_t plane_in = (int64_t)d.H * d.W;
    // 16-byte weight loads need every block's run to start on a 16-byte boundary
    const bool w_vec = ((reinterpret_cast<uintptr_t>(weight) & 15u) == 0) && (((int64_t)d.C * taps) & 3) == 0 && ((rc_block * taps) & 3) == 0;
    for (int c0 = 0; c0 < d.C; c0 += rc_block) {
        const int nrc = (d.C - c0) < rc_block ? (d.C - c0) : rc_block;
        __syncthreads();  // the previous block of weights has been used
        // A channel's nrc * taps weights of this block are contiguous in the OIHW tensor. Consecutive threads take
        // consecutive channels (distinct shared-memory banks) and 16 bytes each where the run allows it: with 4-byte
        // loads every value costs a 32-byte sector of its own, which made the 512-channel layers weight-bound.
        const int run = nrc * taps;
        if (w_vec && (run & 3) == 0) {
            for (int i = threadIdx.x; i < (run >> 2) * kTileO; i += kTileThreads) {
                const int o = i % kTileO, jq = i / kTileO;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (o0 + o < d.O) v = __ldg(reinterpret_cast<const float4*>(weight + ((int64_t)(o0 + o) * d.C + c0) * taps) + jq);
                float* dst = w_s + (4 * jq) * kTileO + o;
                dst[0] = v.x; dst[kTileO] = v.y; dst[2 * kTileO] = v.z; dst[3 * kTileO] = v.w;
            }
        } else {
            for (int i = threadIdx.x; i < run * kTileO; i += kTileThreads) {
                const int o = i % kTileO, j = i / kTileO;
                w_s[i] = (o0 + o < d.O) ? __ldg(weight + ((int64_t)(o0 + o) * d.C + c0) * taps + j) : 0.0f;
            }
        }
        __syncthreads();
        for (int rc = 0; rc < nrc; ++rc) {
            const float* wr = w_s + (rc * taps) * kTileO + og * kOT;
            for (int rh = 0; rh < d.KH; ++rh) {
                const float* row[kPT];
                bool row_ok[kPT];
#pragma unroll
                for (int e = 0; e < kPT; ++e) {
                    const int ih = ih0[e] + rh * d.DH;
                    row_ok[e] = pix_ok[e] && ih >= 0 && ih < d.H;
                    row[e] = xn[e] + (int64_t)(c0 + rc) * plane_in + (int64_t)(row_ok[e] ? ih : 0) * d.W;
                }
#pragma unroll
                for (int rw = 0; rw < KW; ++rw) {
                    float x[kPT];
#pragma unroll
                    for (int e = 0; e < kPT; ++e) {
                        const int iw = iw0[e] + rw * d.DW;
                        x[e] = (row_ok[e] && iw >= 0 && iw < d.W) ? __ldg(row[e] + iw) : 0.0f;
                    }
                    float w[kOT];
#pragma unroll
                    for (int v = 0; v < kOT / 4; ++v) {
                        const float4 wv = *reinterpret_cast<const float4*>(wr + (rh * KW + rw) * kTileO + 4 * v);
                        w[4 * v] = wv.x; w[4 * v + 1] = wv.y; w[4 * v + 2] = wv.z; w[4 * v + 3] = wv.w;
                    }
#pragma unroll
                    for (int j = 0; j < kOT; ++j)
#pragma unroll
                        for (int e = 0; e < kPT; ++e) acc[j][e] = __fadd_rn(acc[j][e], __fmul_rn(x[e], w[j]));
                }
            }
        }
    }
#pragma unroll
    for (int e = 0; e < kPT; ++e) {
        const int64_t p = p0 + pg + kPG * e;
        if (p >= P) continue;
        const int64_t n = p / plane_out, rem = p - n * plane_out;
#pragma unroll
        for (int j = 0; j < kOT; ++j) {
            const int o = o0 + og * kOT + j;
            if (o < d.O) epi(acc[j][e], (n * d.O + o) * plane_out + rem, o);
        }
    }
}

template <int kOT, int kPT, typename Epilogue>
void launch_tiled_f32(const float* data, const float* weight, const ConvDims& d, int rc_block, const Epilogue& epi, cudaStream_t s) {
    constexpr int kTileP = (kTileThreads / (kTileO / kOT)) * kPT;
    const int64_t P = (int64_t)d.N * d.OH * d.OW;
    const dim3 grid((unsigned)((P + kTileP - 1) / kTileP), (unsigned)((d.O + kTileO - 1) / kTileO), 1u);
    const size_t smem = (size_t)rc_block * d.KH * d.KW * kTileO * sizeof(float);
    switch (d.KW) {
        case 1: conv2d_tiled_f32_kernel<1, kOT, kPT, Epilogue><<<grid, kTileThreads, smem, s>>>(data, weight, d, rc_block, epi); break;
        case 3: conv2d_tiled_f32_kernel<3, kOT, kPT, Epilogue><<<grid, kTileThreads, smem, s>>>(data, weight, d, rc_block, epi); break;
        case 7: conv2d_tiled_f32_kernel<7, kOT, kPT, Epilogue><<<grid, kTileThreads, smem, s>>>(data, weight, d, rc_block, epi); break;
        default: conv2d_tiled_f32_kernel<0, kOT, kPT, Epilogue><<<grid, kTileThreads, smem, s>>>(data, weight, d, rc_block, epi); break;
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
    const int taps = d.KH * d.KW;
    // weights of up to 8 input channels per shared-memory block, within 40 KiB
    int rc_block = (40 * 1024) / (taps * kTileO * (int)sizeof(float));
    if (rc_block > 8) rc_block = 8;
    if (rc_block > d.C) rc_block = d.C;
    // the tiled kernel for anything that fills a few blocks; tiny problems and huge filters stay with one thread per output
    const int64_t pixels = (int64_t)d.N * d.OH * d.OW;
    if (rc_block >= 1 && total >= 4096 && (pixels + 15) / 16 <= 0x7fffffffll && (d.O + kTileO - 1) / kTileO <= 65535) {
        // (a 4 x 2 shape with four times as many threads for the deep layers of a small batch was measured slower:
        // 1.78 / 1.94 ms against 1.13 / 1.52 ms on the layer-3 / layer-4 convolutions of ResNet-18 at 32 images)
        launch_tiled_f32<8, 4>(data, weight, d, rc_block, epi, s);
        return check_launch("nn_conv2d (fp32, tiled)");
    }
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

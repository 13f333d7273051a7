// Kernels of the whole-graph executor that work on its internal activation format: NHWC
// (channel-innermost), bf16 or fp32 storage. All HBM-bound: 16-byte vector accesses along the
// channel axis, grids sized as a multiple of the SM count.
//
// Semantics follow the reference ops exactly on the stored values:
//   max pool  m = -inf; v = inb ? x : -1e30f; m = (m > v) ? m : v  (include/te/topi/nn.h:161-229)
//   gap       s = 0; s = s + x over (h, w) in order; s / (float)(H*W)  (include/te/topi/nn.h:260-287)
//   add/relu  one fp32 add, `x > 0 ? x : 0`  (include/te/topi/broadcast.h:90-109, nn.h:19-30)
// with bf16 storage rounding (nearest even) applied when a result is written back as bf16.
#include "nhwc_kernels.cuh"

#include <cuda_bf16.h>

#include <algorithm>
#include <cmath>

#include "common.cuh"
#include "sm100.cuh"

namespace kxc_b200 {
namespace {

constexpr int kThreads = 256;

// 16-byte vector of activations <-> fp32 lanes
template <typename T>
struct Vec;
template <>
struct Vec<__nv_bfloat16> {
    static constexpr int kLanes = 8;
    __device__ static void load(const __nv_bfloat16* p, float (&f)[8]) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            f[2 * k] = __uint_as_float(w[k] << 16);
            f[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
        }
    }
    __device__ static void store(__nv_bfloat16* p, const float (&f)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
            w[k] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};
template <>
struct Vec<float> {
    static constexpr int kLanes = 4;
    __device__ static void load(const float* p, float (&f)[4]) {
        const float4 u = __ldg(reinterpret_cast<const float4*>(p));
        f[0] = u.x; f[1] = u.y; f[2] = u.z; f[3] = u.w;
    }
    // fp32 storage holds tf32 operands: every stored activation is rounded (nearest even) to the 10-bit
    // mantissa the tensor cores read, so that what the next contraction sees is well defined
    __device__ static float rnd(float x) {
        uint32_t u = __float_as_uint(x);
        if ((u & 0x7f800000u) != 0x7f800000u) u = (u + 0xfffu + ((u >> 13) & 1u)) & 0xffffe000u;
        return __uint_as_float(u);
    }
    __device__ static void store(float* p, const float (&f)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(rnd(f[0]), rnd(f[1]), rnd(f[2]), rnd(f[3]));
    }
};

template <typename T>
__global__ void __launch_bounds__(kThreads) maxpool_nhwc_kernel(const T* __restrict__ x, T* __restrict__ out, int N, int H,
                                                                int W, int C, int OH, int OW, int KH, int KW, int SH, int SW,
                                                                int PT, int PL) {
    constexpr int L = Vec<T>::kLanes;
    const int cg = C / L;
    const int64_t total = (int64_t)N * OH * OW * cg;
    for (int64_t lin = (int64_t)blockIdx.x * kThreads + threadIdx.x; lin < total; lin += (int64_t)gridDim.x * kThreads) {
        const int g = (int)(lin % cg);
        int64_t t = lin / cg;
        const int ow = (int)(t % OW); t /= OW;
        const int oh = (int)(t % OH);
        const int n = (int)(t / OH);
        float m[L];
#pragma unroll
        for (int j = 0; j < L; ++j) m[j] = -INFINITY;
        for (int rh = 0; rh < KH; ++rh) {
            const int ih = oh * SH + rh - PT;
            for (int rw = 0; rw < KW; ++rw) {
                const int iw = ow * SW + rw - PL;
                float v[L];
                if (ih >= 0 && ih < H && iw >= 0 && iw < W) {
                    Vec<T>::load(x + (((int64_t)n * H + ih) * W + iw) * C + g * L, v);
                } else {
#pragma unroll
                    for (int j = 0; j < L; ++j) v[j] = -1e30f;
                }
#pragma unroll
                for (int j = 0; j < L; ++j) m[j] = (m[j] > v[j]) ? m[j] : v[j];
            }
        }
        Vec<T>::store(out + lin * L, m);
    }
}

// 3x3 window, stride 2, padding 1, even OH/OW: a thread produces a 2x2 block of outputs for one channel
// vector from the 5x5 input window, walking the window ONCE in row-major order. Every one of the four
// accumulators thereby still sees its own nine taps in the reference's rh -> rw order (bit-exact,
// NaN handling included), with 25 loads per 4 outputs instead of 36.
template <typename T>
__global__ void __launch_bounds__(kThreads) maxpool3x3s2p1_nhwc_kernel(const T* __restrict__ x, T* __restrict__ out, int N, int H,
                                                                       int W, int C, int OH, int OW) {
    constexpr int L = Vec<T>::kLanes;
    const int cg = C / L, ow2n = OW / 2, oh2n = OH / 2;
    const int64_t total = (int64_t)N * oh2n * ow2n * cg;
    for (int64_t lin = (int64_t)blockIdx.x * kThreads + threadIdx.x; lin < total; lin += (int64_t)gridDim.x * kThreads) {
        const int g = (int)(lin % cg);
        int64_t t = lin / cg;
        const int ow2 = (int)(t % ow2n); t /= ow2n;
        const int oh2 = (int)(t % oh2n);
        const int n = (int)(t / oh2n);
        float m[2][2][L];
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int b = 0; b < 2; ++b)
#pragma unroll
                for (int j = 0; j < L; ++j) m[a][b][j] = -INFINITY;
        const T* base = x + (int64_t)n * H * W * C + g * L;
#pragma unroll
        for (int ir = 0; ir < 5; ++ir) {
            const int ih = 4 * oh2 - 1 + ir;
            const bool row_ok = ih >= 0 && ih < H;
#pragma unroll
            for (int ic = 0; ic < 5; ++ic) {
                const int iw = 4 * ow2 - 1 + ic;
                float v[L];
                if (row_ok && iw >= 0 && iw < W) {
                    Vec<T>::load(base + ((int64_t)ih * W + iw) * C, v);
                } else {
#pragma unroll
                    for (int j = 0; j < L; ++j) v[j] = -1e30f;
                }
                // input (ir, ic) is tap (ir - 2a, ic - 2b) of output (a, b) when both offsets are in [0, 2]
#pragma unroll
                for (int a = 0; a < 2; ++a)
#pragma unroll
                    for (int b = 0; b < 2; ++b)
                        if (ir - 2 * a >= 0 && ir - 2 * a <= 2 && ic - 2 * b >= 0 && ic - 2 * b <= 2) {
#pragma unroll
                            for (int j = 0; j < L; ++j) m[a][b][j] = (m[a][b][j] > v[j]) ? m[a][b][j] : v[j];
                        }
            }
        }
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int b = 0; b < 2; ++b)
                Vec<T>::store(out + ((((int64_t)n * OH + 2 * oh2 + a) * OW + 2 * ow2 + b) * C) + g * L, m[a][b]);
    }
}

// Global average over the pixels of NHWC activations, the pixels of an (image, channel group) dealt to the block's
// eight warps: every warp sums its pixels (all loads in flight at once), the partial sums meet in shared memory and
// are added in warp order. The summation order differs from the reference's sequential walk (tensor-core plans
// compare with a tolerance; the bit-exact fp32 plan uses the NCHW kernel in pool.cu).
template <typename T>
__global__ void __launch_bounds__(kThreads) gap_nhwc_split_kernel(const T* __restrict__ x, T* __restrict__ out, int N, int HW,
                                                                  int C) {
    constexpr int L = Vec<T>::kLanes;
    constexpr int kParts = kThreads / 32;
    __shared__ float part_sum[kParts][32][L];
    const int cg = C / L;
    const int64_t total = (int64_t)N * cg;
    const int lane = threadIdx.x & 31, part = threadIdx.x >> 5;
    const float div = (float)HW;
    sm100::pdl_launch_dependents();
    sm100::pdl_wait();
    for (int64_t base = (int64_t)blockIdx.x * 32; base < total; base += (int64_t)gridDim.x * 32) {
        const int64_t lin = base + lane;
        float s[L];
#pragma unroll
        for (int j = 0; j < L; ++j) s[j] = 0.0f;
        if (lin < total) {
            const int g = (int)(lin % cg);
            const int n = (int)(lin / cg);
            const T* p = x + (int64_t)n * HW * C + g * L;
            for (int i0 = part; i0 < HW; i0 += 8 * kParts) {
                float v[8][L];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int i = i0 + u * kParts;
                    if (i < HW) {
                        Vec<T>::load(p + (int64_t)i * C, v[u]);
                    } else {
#pragma unroll
                        for (int j = 0; j < L; ++j) v[u][j] = 0.0f;
                    }
                }
#pragma unroll
                for (int u = 0; u < 8; ++u)
#pragma unroll
                    for (int j = 0; j < L; ++j) s[j] = __fadd_rn(s[j], v[u][j]);
            }
        }
#pragma unroll
        for (int j = 0; j < L; ++j) part_sum[part][lane][j] = s[j];
        __syncthreads();
        if (part == 0 && lin < total) {
#pragma unroll
            for (int q = 1; q < kParts; ++q)
#pragma unroll
                for (int j = 0; j < L; ++j) s[j] = __fadd_rn(s[j], part_sum[q][lane][j]);
#pragma unroll
            for (int j = 0; j < L; ++j) s[j] = __fdiv_rn(s[j], div);
            Vec<T>::store(out + lin * L, s);
        }
        __syncthreads();
    }
}

// out = relu?(a (+ b)) on flat arrays of the same shape; b may be null (plain relu)
template <typename T>
__global__ void __launch_bounds__(kThreads) eltwise_nhwc_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                                T* __restrict__ out, int64_t nvec, int relu) {
    constexpr int L = Vec<T>::kLanes;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * kThreads) {
        float va[L];
        Vec<T>::load(a + i * L, va);
        if (b != nullptr) {
            float vb[L];
            Vec<T>::load(b + i * L, vb);
#pragma unroll
            for (int j = 0; j < L; ++j) va[j] = __fadd_rn(va[j], vb[j]);
        }
        if (relu) {
#pragma unroll
            for (int j = 0; j < L; ++j) va[j] = va[j] > 0.0f ? va[j] : 0.0f;
        }
        Vec<T>::store(out + i * L, va);
    }
}

// NHWC (bf16/fp32) -> NCHW fp32 through a shared-memory transpose tile; grid (ceil(HW/32), ceil(C/32), N)
template <typename T>
__global__ void nhwc_to_nchw_kernel(const T* __restrict__ in, float* __restrict__ out, int C, int HW) {
    __shared__ float tile[32][33];
    const int n = blockIdx.z, hw0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    const T* src = in + (size_t)n * HW * C;
    float* dst = out + (size_t)n * C * HW;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int hw = hw0 + threadIdx.y + 8 * k, c = c0 + threadIdx.x;
        tile[threadIdx.y + 8 * k][threadIdx.x] = (hw < HW && c < C) ? (float)src[(size_t)hw * C + c] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int c = c0 + threadIdx.y + 8 * k, hw = hw0 + threadIdx.x;
        if (c < C && hw < HW) dst[(size_t)c * HW + hw] = tile[threadIdx.x][threadIdx.y + 8 * k];
    }
}

__device__ __forceinline__ float round_tf32_rne(float x) {
    uint32_t u = __float_as_uint(x);
    if ((u & 0x7f800000u) != 0x7f800000u) u = (u + 0xfffu + ((u >> 13) & 1u)) & 0xffffe000u;
    return __uint_as_float(u);
}
template <typename T>
__device__ __forceinline__ T to_operand(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 to_operand<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ float to_operand<float>(float v) { return round_tf32_rne(v); }

// Stem input packing: NCHW fp32 [N,C<=4,H,W] -> [N][H+2*pad_h][Wp][4] operand type with a zero border,
// so that the 8 consecutive pixels x 4 channels starting at an even column form one K block.
template <typename T>
__global__ void __launch_bounds__(kThreads) stem_pack_kernel(const float* __restrict__ x, T* __restrict__ out, int N, int C,
                                                             int H, int W, int Hp, int Wp, int pad_h, int pad_w) {
    // four consecutive packed pixels per thread (Wp is a multiple of 4): 12 independent loads in flight,
    // 32 or 64 contiguous bytes stored
    const int wq = Wp / 4;
    const int64_t total = (int64_t)N * Hp * wq;
    sm100::pdl_launch_dependents();
    sm100::pdl_wait();  // the packed buffer may still be read by a kernel of the previous run
    for (int64_t lin = (int64_t)blockIdx.x * kThreads + threadIdx.x; lin < total; lin += (int64_t)gridDim.x * kThreads) {
        const int wp0 = (int)(lin % wq) * 4;
        int64_t t = lin / wq;
        const int hp = (int)(t % Hp);
        const int n = (int)(t / Hp);
        const int h = hp - pad_h;
        const bool row_ok = h >= 0 && h < H;
        float f[4][4];
#pragma unroll
        for (int px = 0; px < 4; ++px) {
            const int w = wp0 + px - pad_w;
#pragma unroll
            for (int c = 0; c < 4; ++c)
                f[px][c] = (c < C && row_ok && w >= 0 && w < W) ? __ldg(x + (((int64_t)n * C + c) * H + h) * W + w) : 0.0f;
        }
        T v[16];
#pragma unroll
        for (int px = 0; px < 4; ++px)
#pragma unroll
            for (int c = 0; c < 4; ++c) v[px * 4 + c] = to_operand<T>(f[px][c]);
        T* dst = out + (((int64_t)n * Hp + hp) * Wp + wp0) * 4;
        constexpr int kVecs = (int)(sizeof(T) * 16 / 16);
#pragma unroll
        for (int q = 0; q < kVecs; ++q) reinterpret_cast<uint4*>(dst)[q] = reinterpret_cast<const uint4*>(v)[q];
    }
}

// Stem weights: OIHW fp32 [O,C<=4,KH,KW<=8] -> [O][KH][8][4] operand type, zero for kw >= KW or c >= C
template <typename T>
__global__ void stem_pack_weights_kernel(const float* __restrict__ w, T* __restrict__ out, int O, int C, int KH, int KW) {
    const int total = O * KH * 32;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int c = i & 3, kw = (i >> 2) & 7;
        const int kh = (i >> 5) % KH, o = (i >> 5) / KH;
        float f = 0.0f;
        if (c < C && kw < KW) f = w[((o * C + c) * KH + kh) * KW + kw];
        out[i] = to_operand<T>(f);
    }
}

int grid_for(int64_t items, int per_sm = 8) {
    int64_t b = (items + kThreads - 1) / kThreads;
    const int64_t cap = (int64_t)kNumSMs * per_sm;
    if (b > cap) b = cap;
    if (b < 1) b = 1;
    return (int)b;
}

}  // namespace

#define KXC_DISPATCH_ACT(dtype, ...)                         \
    if ((dtype) == kTcBF16) {                                \
        using T = __nv_bfloat16;                             \
        __VA_ARGS__;                                         \
    } else if ((dtype) == kTcTF32) {                         \
        using T = float;                                     \
        __VA_ARGS__;                                         \
    } else {                                                 \
        return fail(KXC_B200_ERR_INVALID, "activation dtype"); \
    }

int32_t maxpool_nhwc(const void* x, void* out, TcDType dt, int N, int H, int W, int C, int OH, int OW, int KH, int KW, int SH,
                     int SW, int PT, int PL, cudaStream_t s) {
    const int lanes = dt == kTcBF16 ? 8 : 4;
    if (C % lanes != 0) return fail(KXC_B200_ERR_UNSUPPORTED, "NHWC max pool: %d channels is not a multiple of %d", C, lanes);
    const int64_t items = (int64_t)N * OH * OW * (C / lanes);
    if (items == 0) return KXC_B200_OK;
    if (KH == 3 && KW == 3 && SH == 2 && SW == 2 && PT == 1 && PL == 1 && (OH % 2) == 0 && (OW % 2) == 0 && OH == (H + 2 - 3) / 2 + 1 &&
        OW == (W + 2 - 3) / 2 + 1) {
        KXC_DISPATCH_ACT(dt, (maxpool3x3s2p1_nhwc_kernel<T><<<grid_for(items / 4, 16), kThreads, 0, s>>>(
                                 static_cast<const T*>(x), static_cast<T*>(out), N, H, W, C, OH, OW)));
        return check_launch("maxpool3x3s2p1_nhwc");
    }
    KXC_DISPATCH_ACT(dt, (maxpool_nhwc_kernel<T><<<grid_for(items, 16), kThreads, 0, s>>>(
                             static_cast<const T*>(x), static_cast<T*>(out), N, H, W, C, OH, OW, KH, KW, SH, SW, PT, PL)));
    return check_launch("maxpool_nhwc");
}

int32_t gap_nhwc(const void* x, void* out, TcDType dt, int N, int HW, int C, cudaStream_t s) {
    const int lanes = dt == kTcBF16 ? 8 : 4;
    if (C % lanes != 0) return fail(KXC_B200_ERR_UNSUPPORTED, "NHWC global pool: %d channels is not a multiple of %d", C, lanes);
    const int64_t items = (int64_t)N * (C / lanes);
    if (items == 0) return KXC_B200_OK;
    cudaError_t err = cudaSuccess;
    const int blocks = (int)std::min<int64_t>((items + 31) / 32, (int64_t)kNumSMs * 16);
    KXC_DISPATCH_ACT(dt, (err = launch_kernel(gap_nhwc_split_kernel<T>, dim3(blocks), dim3(kThreads), 0, s, /*pdl=*/true, 1,
                                              static_cast<const T*>(x), static_cast<T*>(out), N, HW, C)));
    if (err != cudaSuccess) return fail(KXC_B200_ERR_CUDA, "gap_nhwc launch: %s", cudaGetErrorString(err));
    return check_launch("gap_nhwc");
}

int32_t eltwise_nhwc(const void* a, const void* b, void* out, TcDType dt, int64_t numel, int relu, cudaStream_t s) {
    const int lanes = dt == kTcBF16 ? 8 : 4;
    if (numel % lanes != 0) return fail(KXC_B200_ERR_UNSUPPORTED, "NHWC elementwise: %lld elements is not a multiple of %d", (long long)numel, lanes);
    const int64_t nvec = numel / lanes;
    if (nvec == 0) return KXC_B200_OK;
    KXC_DISPATCH_ACT(dt, (eltwise_nhwc_kernel<T><<<grid_for(nvec, 16), kThreads, 0, s>>>(
                             static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out), nvec, relu)));
    return check_launch("eltwise_nhwc");
}

int32_t nhwc_to_nchw_f32(const void* in, float* out, TcDType dt, int N, int C, int HW, cudaStream_t s) {
    if (N == 0) return KXC_B200_OK;
    if (N > 65535) return fail(KXC_B200_ERR_UNSUPPORTED, "layout transform: batch %d exceeds the grid limit", N);
    const dim3 grid((HW + 31) / 32, (C + 31) / 32, N), block(32, 8);
    KXC_DISPATCH_ACT(dt, (nhwc_to_nchw_kernel<T><<<grid, block, 0, s>>>(static_cast<const T*>(in), out, C, HW)));
    return check_launch("nhwc_to_nchw");
}

int32_t stem_pack(const float* x, void* out, TcDType dt, int N, int C, int H, int W, int Hp, int Wp, int pad_h, int pad_w,
                  cudaStream_t s) {
    if (Wp % 4 != 0) return fail(KXC_B200_ERR_INVALID, "stem_pack: packed width %d must be a multiple of 4", Wp);
    const int64_t items = (int64_t)N * Hp * (Wp / 4);
    if (items == 0) return KXC_B200_OK;
    cudaError_t err = cudaSuccess;
    KXC_DISPATCH_ACT(dt, (err = launch_kernel(stem_pack_kernel<T>, dim3(grid_for(items, 16)), dim3(kThreads), 0, s, /*pdl=*/true, 1, x,
                                              static_cast<T*>(out), N, C, H, W, Hp, Wp, pad_h, pad_w)));
    if (err != cudaSuccess) return fail(KXC_B200_ERR_CUDA, "stem_pack launch: %s", cudaGetErrorString(err));
    return check_launch("stem_pack");
}

int32_t stem_pack_weights(const float* w, void* out, TcDType dt, int O, int C, int KH, int KW, cudaStream_t s) {
    KXC_DISPATCH_ACT(dt, (stem_pack_weights_kernel<T><<<grid_for((int64_t)O * KH * 32), kThreads, 0, s>>>(w, static_cast<T*>(out), O,
                                                                                                          C, KH, KW)));
    return check_launch("stem_pack_weights");
}

}  // namespace kxc_b200

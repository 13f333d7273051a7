// Layout / precision conversion kernels (HBM-bound, coalesced on both sides through a shared-memory
// transpose tile).
#include "layout.cuh"

#include <cuda_bf16.h>

#include "common.cuh"

namespace kxc_b200 {
namespace {

__device__ __forceinline__ float round_tf32_rne(float x) {
    uint32_t u = __float_as_uint(x);
    if ((u & 0x7f800000u) != 0x7f800000u) u = (u + 0xfffu + ((u >> 13) & 1u)) & 0xffffe000u;
    return __uint_as_float(u);
}

template <typename TOut>
__device__ __forceinline__ TOut convert_to(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 convert_to<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ float convert_to<float>(float v) { return round_tf32_rne(v); }

// What single-pass tf32 drops: the tf32 rounding of (v - tf32(v)). a*b ~ a_hi*b_hi + a_hi*b_lo + a_lo*b_hi then carries
// about 21 bits of each operand instead of 11.
struct Tf32Lo {
    float v;
};
template <>
__device__ __forceinline__ Tf32Lo convert_to<Tf32Lo>(float v) {
    const float hi = round_tf32_rne(v);
    // inf - inf would be NaN: a non-finite value lives in the high part only
    return Tf32Lo{(__float_as_uint(v) & 0x7f800000u) == 0x7f800000u ? 0.0f : round_tf32_rne(__fsub_rn(v, hi))};
}

template <typename TIn, typename TOut>
__device__ __forceinline__ TOut convert_elem(TIn v) { return convert_to<TOut>((float)v); }
template <>
__device__ __forceinline__ int8_t convert_elem<int8_t, int8_t>(int8_t v) { return v; }

// grid (ceil(HW/32), ceil(cpad/32), N), block (32, 8)
template <typename TIn, typename TOut>
__global__ void nchw_to_nhwc_kernel(const TIn* __restrict__ in, TOut* __restrict__ out, int C, int HW, int cpad) {
    __shared__ TIn tile[32][33];
    const int n = blockIdx.z;
    const int hw0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    const TIn* src = in + (size_t)n * C * HW;
    TOut* dst = out + (size_t)n * HW * cpad;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int c = c0 + threadIdx.y + 8 * k, hw = hw0 + threadIdx.x;
        tile[threadIdx.y + 8 * k][threadIdx.x] = (c < C && hw < HW) ? src[(size_t)c * HW + hw] : (TIn)0;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int hw = hw0 + threadIdx.y + 8 * k, c = c0 + threadIdx.x;
        if (hw < HW && c < cpad) dst[(size_t)hw * cpad + c] = convert_elem<TIn, TOut>(tile[threadIdx.x][threadIdx.y + 8 * k]);
    }
}

// int8 form: 64 channels x 64 pixels per block, four bytes per thread on both sides (64-byte runs in HBM instead of the
// 32-byte runs the element-wise kernel makes of 1-byte elements). grid (ceil(HW/64), ceil(cpad/64), N), block 256.
// It is a batched byte transpose [C][HW] -> [HW][cpad] (rows c >= C read as zero), so it also serves NHWC -> NCHW with
// the roles of the two extents exchanged; vec_out = 0 when the destination rows are not 4-byte multiples.
__global__ void __launch_bounds__(256) nchw_to_nhwc_s8_kernel(const int8_t* __restrict__ in, int8_t* __restrict__ out, int C, int HW,
                                                               int cpad, int vec_in, int vec_out) {
    __shared__ __align__(4) int8_t tile[64][68];
    const int n = blockIdx.z;
    const int hw0 = blockIdx.x * 64, c0 = blockIdx.y * 64;
    const int8_t* src = in + (size_t)n * C * HW;
    int8_t* dst = out + (size_t)n * HW * cpad;
    const int q = threadIdx.x & 15, r = threadIdx.x >> 4;  // 16 four-byte columns x 16 rows per pass
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int c = c0 + r + 16 * k, hw = hw0 + 4 * q;
        uint32_t v = 0;
        if (c < C) {
            const int8_t* s4 = src + (size_t)c * HW + hw;
            if (vec_in && hw + 3 < HW) {
                v = __ldg(reinterpret_cast<const uint32_t*>(s4));
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (hw + e < HW) v |= (uint32_t)(uint8_t)__ldg(s4 + e) << (8 * e);
            }
        }
        *reinterpret_cast<uint32_t*>(&tile[r + 16 * k][4 * q]) = v;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int hw = hw0 + r + 16 * k, c = c0 + 4 * q;
        if (hw < HW && c < cpad) {
            const int hl = r + 16 * k;
            const uint32_t v = (uint32_t)(uint8_t)tile[4 * q][hl] | ((uint32_t)(uint8_t)tile[4 * q + 1][hl] << 8) |
                               ((uint32_t)(uint8_t)tile[4 * q + 2][hl] << 16) | ((uint32_t)(uint8_t)tile[4 * q + 3][hl] << 24);
            int8_t* d4 = dst + (size_t)hw * cpad + c;
            if (vec_out) {  // cpad is a multiple of 4: the four bytes are in or out together
                *reinterpret_cast<uint32_t*>(d4) = v;
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (c + e < cpad) d4[e] = (int8_t)(v >> (8 * e));
            }
        }
    }
}

// int8 NCHW -> NHWC of the pixels a 1x1 convolution of stride `st` (no padding) reads: out[n][p][c] =
// in[n][c][(p / OW) * st][(p % OW) * st], p = oh * OW + ow. grid (ceil(OH*OW/64), ceil(cpad/64), N), block 256: the same
// 64 x 64 byte transpose as above with gathered source pixels; the rows the convolution skips are never touched.
__global__ void __launch_bounds__(256) nchw_to_nhwc_s8_subsample_kernel(const int8_t* __restrict__ in, int8_t* __restrict__ out, int C,
                                                                         int H, int W, int OH, int OW, int st, int cpad) {
    __shared__ __align__(4) int8_t tile[64][68];
    const int n = blockIdx.z;
    const int p0 = blockIdx.x * 64, c0 = blockIdx.y * 64;
    const int P = OH * OW;
    const int8_t* src = in + (size_t)n * C * H * W;
    int8_t* dst = out + (size_t)n * P * cpad;
    const int q = threadIdx.x & 15, r = threadIdx.x >> 4;
    int off[4];  // source offsets of this thread's four pixels inside a channel plane (-1: beyond the last pixel)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const int p = p0 + 4 * q + e;
        off[e] = p < P ? (p / OW) * st * W + (p % OW) * st : -1;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int c = c0 + r + 16 * k;
        uint32_t v = 0;
        if (c < C) {
            const int8_t* plane = src + (size_t)c * H * W;
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (off[e] >= 0) v |= (uint32_t)(uint8_t)__ldg(plane + off[e]) << (8 * e);
        }
        *reinterpret_cast<uint32_t*>(&tile[r + 16 * k][4 * q]) = v;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int p = p0 + r + 16 * k, c = c0 + 4 * q;
        if (p < P && c < cpad) {  // cpad is a multiple of 4
            const int pl = r + 16 * k;
            const uint32_t v = (uint32_t)(uint8_t)tile[4 * q][pl] | ((uint32_t)(uint8_t)tile[4 * q + 1][pl] << 8) |
                               ((uint32_t)(uint8_t)tile[4 * q + 2][pl] << 16) | ((uint32_t)(uint8_t)tile[4 * q + 3][pl] << 24);
            *reinterpret_cast<uint32_t*>(dst + (size_t)p * cpad + c) = v;
        }
    }
}

template <typename TIn, typename TOut>
__global__ void pack_weights_kernel(const TIn* __restrict__ w, TOut* __restrict__ out, int O, int C, int KH, int KW, int cpad) {
    const int64_t total = (int64_t)O * KH * KW * cpad;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % cpad);
        int64_t t = i / cpad;
        const int kw = (int)(t % KW); t /= KW;
        const int kh = (int)(t % KH);
        const int o = (int)(t / KH);
        out[i] = c < C ? convert_elem<TIn, TOut>(w[(((int64_t)o * C + c) * KH + kh) * KW + kw]) : convert_elem<TIn, TOut>((TIn)0);
    }
}

template <typename TOut>
__global__ void convert_rows_kernel(const float* __restrict__ in, TOut* __restrict__ out, int64_t rows, int cols, int cpad) {
    const int64_t total = rows * cpad;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % cpad);
        const int64_t r = i / cpad;
        out[i] = convert_to<TOut>(c < cols ? in[r * cols + c] : 0.0f);
    }
}

int grid_1d(int64_t items, int threads) {
    int64_t b = (items + threads - 1) / threads;
    const int64_t cap = (int64_t)kNumSMs * 16;
    if (b > cap) b = cap;
    if (b < 1) b = 1;
    return (int)b;
}

}  // namespace

int32_t nchw_to_nhwc(const void* in, void* out, TcDType dtype, int N, int C, int HW, int cpad, cudaStream_t s, bool tf32_lo) {
    if (N == 0) return KXC_B200_OK;
    if (N > 65535) return fail(KXC_B200_ERR_UNSUPPORTED, "layout transform: batch %d exceeds the grid limit", N);
    const dim3 grid((HW + 31) / 32, (cpad + 31) / 32, N), block(32, 8);
    switch (dtype) {
        case kTcBF16:
            nchw_to_nhwc_kernel<float, __nv_bfloat16><<<grid, block, 0, s>>>(static_cast<const float*>(in), static_cast<__nv_bfloat16*>(out), C, HW, cpad);
            break;
        case kTcTF32:
            if (tf32_lo)
                nchw_to_nhwc_kernel<float, Tf32Lo><<<grid, block, 0, s>>>(static_cast<const float*>(in), static_cast<Tf32Lo*>(out), C, HW, cpad);
            else
                nchw_to_nhwc_kernel<float, float><<<grid, block, 0, s>>>(static_cast<const float*>(in), static_cast<float*>(out), C, HW, cpad);
            break;
        case kTcS8:
            if ((cpad & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 3u) == 0) {
                const int vec_in = ((HW & 3) == 0 && (reinterpret_cast<uintptr_t>(in) & 3u) == 0) ? 1 : 0;
                nchw_to_nhwc_s8_kernel<<<dim3((HW + 63) / 64, (cpad + 63) / 64, N), 256, 0, s>>>(static_cast<const int8_t*>(in),
                                                                                                static_cast<int8_t*>(out), C, HW, cpad, vec_in, 1);
            } else {
                nchw_to_nhwc_kernel<int8_t, int8_t><<<grid, block, 0, s>>>(static_cast<const int8_t*>(in), static_cast<int8_t*>(out), C, HW, cpad);
            }
            break;
    }
    return check_launch("nchw_to_nhwc");
}

int32_t nchw_to_nhwc_s8_subsample(const int8_t* in, int8_t* out, int N, int C, int H, int W, int OH, int OW, int stride, int cpad,
                                  cudaStream_t s) {
    if (N == 0 || C == 0 || OH == 0 || OW == 0) return KXC_B200_OK;
    if ((cpad & 3) != 0 || (reinterpret_cast<uintptr_t>(out) & 3u) != 0 || N > 65535 || (long long)H * W > 0x7fffffffll)
        return fail(KXC_B200_ERR_UNSUPPORTED, "nchw_to_nhwc_s8_subsample: %d padded channels, %d images", cpad, N);
    nchw_to_nhwc_s8_subsample_kernel<<<dim3((OH * OW + 63) / 64, (cpad + 63) / 64, N), 256, 0, s>>>(in, out, C, H, W, OH, OW, stride, cpad);
    return check_launch("nchw_to_nhwc_s8_subsample");
}

int32_t nhwc_to_nchw_s8(const int8_t* in, int8_t* out, int N, int C, int HW, cudaStream_t s) {
    if (N == 0 || C == 0 || HW == 0) return KXC_B200_OK;
    // source rows = pixels (C bytes each), destination rows = channels (HW bytes each)
    const int vec_in = ((C & 3) == 0 && (reinterpret_cast<uintptr_t>(in) & 3u) == 0) ? 1 : 0;
    const int vec_out = ((HW & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 3u) == 0) ? 1 : 0;
    nchw_to_nhwc_s8_kernel<<<dim3((C + 63) / 64, (HW + 63) / 64, N), 256, 0, s>>>(in, out, HW, C, HW, vec_in, vec_out);
    return check_launch("nhwc_to_nchw_s8");
}

int32_t pack_weights_ohwi(const void* w, void* out, TcDType dtype, int O, int C, int KH, int KW, int cpad, cudaStream_t s, bool tf32_lo) {
    const int64_t total = (int64_t)O * KH * KW * cpad;
    const int grid = grid_1d(total, 256);
    switch (dtype) {
        case kTcBF16:
            pack_weights_kernel<float, __nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const float*>(w), static_cast<__nv_bfloat16*>(out), O, C, KH, KW, cpad);
            break;
        case kTcTF32:
            if (tf32_lo)
                pack_weights_kernel<float, Tf32Lo><<<grid, 256, 0, s>>>(static_cast<const float*>(w), static_cast<Tf32Lo*>(out), O, C, KH, KW, cpad);
            else
                pack_weights_kernel<float, float><<<grid, 256, 0, s>>>(static_cast<const float*>(w), static_cast<float*>(out), O, C, KH, KW, cpad);
            break;
        case kTcS8:
            pack_weights_kernel<int8_t, int8_t><<<grid, 256, 0, s>>>(static_cast<const int8_t*>(w), static_cast<int8_t*>(out), O, C, KH, KW, cpad);
            break;
    }
    return check_launch("pack_weights");
}

int32_t convert_rows(const float* in, void* out, TcDType dtype, int64_t rows, int cols, int cpad, cudaStream_t s, bool tf32_lo) {
    const int64_t total = rows * cpad;
    if (total == 0) return KXC_B200_OK;
    const int grid = grid_1d(total, 256);
    if (dtype == kTcBF16)
        convert_rows_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(in, static_cast<__nv_bfloat16*>(out), rows, cols, cpad);
    else if (dtype == kTcTF32 && tf32_lo)
        convert_rows_kernel<Tf32Lo><<<grid, 256, 0, s>>>(in, static_cast<Tf32Lo*>(out), rows, cols, cpad);
    else if (dtype == kTcTF32)
        convert_rows_kernel<float><<<grid, 256, 0, s>>>(in, static_cast<float*>(out), rows, cols, cpad);
    else
        return fail(KXC_B200_ERR_INVALID, "convert_rows: dtype");
    return check_launch("convert_rows");
}

}  // namespace kxc_b200

// Epilogue code shared by the tensor-core convolution kernels: one thread holds one output pixel's
// 32 consecutive channels (a tcgen05.ld.32x32b.x32 chunk) and applies +bias -> +residual -> ReLU
// (or the int8 requantize) before storing in the requested layout.
#pragma once

#include <cuda_bf16.h>

#include "conv_tc.cuh"

namespace kxc_b200 {

__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Epilogue for one 32-column chunk held by one thread (= one output pixel, 32 consecutive channels).
template <int kOutMode>
__device__ __forceinline__ void epilogue_chunk(const TcParams& p, const uint32_t (&v)[32], int c0, bool valid, int n,
                                               int oh, int ow) {
    if (!valid || c0 >= p.Cout) return;
    const int nch = (p.Cout - c0) < 32 ? (p.Cout - c0) : 32;
    const size_t pix = ((size_t)n * p.OH + oh) * p.OW + ow;

    if constexpr (kOutMode == kOutNHWC_S8 || kOutMode == kOutNCHW_S8) {
        int8_t q[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const int c = c0 + j;
            if (j < nch) {
                const int32_t acc = (int32_t)v[j] + __ldg(p.bias_i32 + c);
                q[j] = requantize_s8(acc, __ldg(p.multiplier + c), __ldg(p.shift + c), p.relu);
            } else {
                q[j] = 0;
            }
        }
        int8_t* out = static_cast<int8_t*>(p.out);
        if constexpr (kOutMode == kOutNHWC_S8) {
            int8_t* dst = out + pix * p.Cout + c0;
            if (nch == 32 && (p.Cout & 15) == 0 && p.vec_ok) {
                const uint4* src = reinterpret_cast<const uint4*>(q);
                reinterpret_cast<uint4*>(dst)[0] = src[0];
                reinterpret_cast<uint4*>(dst)[1] = src[1];
            } else {
                for (int j = 0; j < nch; ++j) dst[j] = q[j];
            }
        } else {
            const size_t plane = (size_t)p.OH * p.OW;
            int8_t* dst = out + ((size_t)n * p.Cout + c0) * plane + (size_t)oh * p.OW + ow;
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < nch) dst[(size_t)j * plane] = q[j];
        }
        return;
    } else {
        float f[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
        if (p.bias != nullptr) {
            if (nch == 32 && p.vec_ok) {
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    const float4 b = __ldg(reinterpret_cast<const float4*>(p.bias + c0 + j));
                    f[j] = __fadd_rn(f[j], b.x);
                    f[j + 1] = __fadd_rn(f[j + 1], b.y);
                    f[j + 2] = __fadd_rn(f[j + 2], b.z);
                    f[j + 3] = __fadd_rn(f[j + 3], b.w);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (j < nch) f[j] = __fadd_rn(f[j], __ldg(p.bias + c0 + j));
            }
        }
        if constexpr (kOutMode == kOutNHWC_BF16) {
            const bool vec = (nch == 32) && ((p.Cout & 7) == 0) && p.vec_ok;
            __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out) + pix * p.Cout + c0;
            if (p.residual != nullptr) {
                const __nv_bfloat16* res = static_cast<const __nv_bfloat16*>(p.residual) + pix * p.Cout + c0;
                if (vec) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const uint4 r = __ldg(reinterpret_cast<const uint4*>(res) + g);
                        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            f[g * 8 + 2 * k] = __fadd_rn(f[g * 8 + 2 * k], bf16_lo(w[k]));
                            f[g * 8 + 2 * k + 1] = __fadd_rn(f[g * 8 + 2 * k + 1], bf16_hi(w[k]));
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (j < nch) f[j] = __fadd_rn(f[j], __bfloat162float(res[j]));
                }
            }
            if (p.relu) {
#pragma unroll
                for (int j = 0; j < 32; ++j) f[j] = f[j] > 0.0f ? f[j] : 0.0f;
            }
            if (vec) {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    uint4 o;
                    o.x = pack_bf16(f[g * 8 + 0], f[g * 8 + 1]);
                    o.y = pack_bf16(f[g * 8 + 2], f[g * 8 + 3]);
                    o.z = pack_bf16(f[g * 8 + 4], f[g * 8 + 5]);
                    o.w = pack_bf16(f[g * 8 + 6], f[g * 8 + 7]);
                    reinterpret_cast<uint4*>(out)[g] = o;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (j < nch) out[j] = __float2bfloat16_rn(f[j]);
            }
        } else if constexpr (kOutMode == kOutNHWC_F32) {
            const bool vec = (nch == 32) && ((p.Cout & 3) == 0) && p.vec_ok;
            float* out = static_cast<float*>(p.out) + pix * p.Cout + c0;
            if (p.residual != nullptr) {
                const float* res = static_cast<const float*>(p.residual) + pix * p.Cout + c0;
                if (vec) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const float4 r = __ldg(reinterpret_cast<const float4*>(res + j));
                        f[j] = __fadd_rn(f[j], r.x);
                        f[j + 1] = __fadd_rn(f[j + 1], r.y);
                        f[j + 2] = __fadd_rn(f[j + 2], r.z);
                        f[j + 3] = __fadd_rn(f[j + 3], r.w);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (j < nch) f[j] = __fadd_rn(f[j], __ldg(res + j));
                }
            }
            if (p.relu) {
#pragma unroll
                for (int j = 0; j < 32; ++j) f[j] = f[j] > 0.0f ? f[j] : 0.0f;
            }
            if (p.round_out_tf32) {  // activation that feeds another tf32 contraction: store what it will read
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    uint32_t u = __float_as_uint(f[j]);
                    if ((u & 0x7f800000u) != 0x7f800000u) u = (u + 0xfffu + ((u >> 13) & 1u)) & 0xffffe000u;
                    f[j] = __uint_as_float(u);
                }
            }
            if (vec) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *reinterpret_cast<float4*>(out + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (j < nch) out[j] = f[j];
            }
        } else {  // kOutNCHW_F32: lanes are consecutive pixels, so each channel's store is contiguous
            const size_t plane = (size_t)p.OH * p.OW;
            const size_t off = ((size_t)n * p.Cout + c0) * plane + (size_t)oh * p.OW + ow;
            float* out = static_cast<float*>(p.out) + off;
            const float* res = p.residual ? static_cast<const float*>(p.residual) + off : nullptr;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if (j < nch) {
                    float x = f[j];
                    if (res) x = __fadd_rn(x, __ldg(res + (size_t)j * plane));
                    if (p.relu) x = x > 0.0f ? x : 0.0f;
                    out[(size_t)j * plane] = x;
                }
            }
        }
    }
}

// Hot-path epilogue (bf16 NHWC activations, channel count a multiple of 32, 16-byte aligned pointers):
// the residual vector is fetched by the caller BEFORE it waits for the accumulator, so its latency
// hides behind the main loop.
__device__ __forceinline__ void epilogue_fast_bf16(const TcParams& p, const uint32_t (&v)[32], int c0, size_t pix,
                                                   const uint4 (&res)[4], bool has_res) {
    float f[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
    if (p.bias != nullptr) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            const float4 b = __ldg(reinterpret_cast<const float4*>(p.bias + c0 + j));
            f[j] = __fadd_rn(f[j], b.x);
            f[j + 1] = __fadd_rn(f[j + 1], b.y);
            f[j + 2] = __fadd_rn(f[j + 2], b.z);
            f[j + 3] = __fadd_rn(f[j + 3], b.w);
        }
    }
    if (has_res) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const uint32_t w[4] = {res[g].x, res[g].y, res[g].z, res[g].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                f[g * 8 + 2 * k] = __fadd_rn(f[g * 8 + 2 * k], bf16_lo(w[k]));
                f[g * 8 + 2 * k + 1] = __fadd_rn(f[g * 8 + 2 * k + 1], bf16_hi(w[k]));
            }
        }
    }
    if (p.relu) {
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = f[j] > 0.0f ? f[j] : 0.0f;
    }
    uint4* out = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + pix * p.Cout + c0);
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        uint4 o;
        o.x = pack_bf16(f[g * 8 + 0], f[g * 8 + 1]);
        o.y = pack_bf16(f[g * 8 + 2], f[g * 8 + 3]);
        o.z = pack_bf16(f[g * 8 + 4], f[g * 8 + 5]);
        o.w = pack_bf16(f[g * 8 + 6], f[g * 8 + 7]);
        out[g] = o;
    }
}

}  // namespace kxc_b200

// Epilogue code shared by the tensor-core convolution kernels: one thread holds one output pixel's
// 32 consecutive channels (a tcgen05.ld.32x32b.x32 chunk) and applies +bias -> +residual -> ReLU
// (or the int8 requantize) before storing in the requested layout.
#pragma once

#include <cuda_bf16.h>

#include <climits>

#include "conv_tc.cuh"

namespace kxc_b200 {

__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// High-word requantize with prepared per-channel constants q = {M, K.lo, K.hi, shift - 1}, K = bias * M + 2^(shift-2+32):
// for 2 <= shift <= 31 (see requant_chunk) and |bias| small enough that acc + bias cannot leave int32,
//   (acc + bias) * M + 2^(S-1) = acc * M + K,   S = 31 + shift,
// so one mad.wide gives the 64-bit sum, its high word shifted by shift-1 is the result before clamping. cvt.pack.sat
// clamps to [-128, 127] and packs two results per instruction; lo_cap = 0 with ReLU, else INT32_MIN (no-op).
// Bytes in channel order.
__device__ __forceinline__ bool requant_prepare(int32_t bias, int32_t mult, int32_t shift, int64_t max_abs_acc, int4* q) {
    const bool ok = (uint32_t)(shift - 2) <= 29u && (int64_t)bias <= (int64_t)INT32_MAX - max_abs_acc &&
                    (int64_t)bias >= (int64_t)INT32_MIN + max_abs_acc;
    const int64_t k = ok ? (int64_t)bias * (int64_t)mult + ((int64_t)1 << (shift - 2 + 32)) : 0;
    *q = make_int4(mult, (int32_t)(uint32_t)(k & 0xffffffffll), (int32_t)(k >> 32), ok ? shift - 1 : 0);
    return ok;
}
__device__ __forceinline__ uint32_t requant4_prepared(const uint32_t (&v)[4], const int4 (&q)[4], int32_t lo_cap) {
    int32_t r[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        int32_t t;
        asm("{\n\t.reg .b64 kk, tt;\n\t.reg .b32 tl;\n\t"
            "mov.b64 kk, {%2, %3};\n\t"
            "mad.wide.s32 tt, %1, %4, kk;\n\t"
            "mov.b64 {tl, %0}, tt;\n\t}"
            : "=r"(t)
            : "r"((int32_t)v[k]), "r"(q[k].y), "r"(q[k].z), "r"(q[k].x));
        t >>= q[k].w;
        r[k] = t < lo_cap ? lo_cap : t;
    }
    uint32_t hi16, out;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi16) : "r"(r[3]), "r"(r[2]), "r"(0));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(r[1]), "r"(r[0]), "r"(hi16));
    return out;
}

// int8 requantize of one chunk: 32 int32 accumulators of consecutive channels c0.. (the first `nch` are real) -> 32 int8
// results, four per word, bytes in channel order.
__device__ __forceinline__ void requant_chunk(const TcParams& p, const uint32_t (&v)[32], int c0, int nch, uint32_t (&qw)[8]) {
    bool done = false;
    if (nch == 32 && p.vec_ok) {
        // Per-channel constants as 16-byte loads (the same addresses in every lane). With 2 <= shift <= 31 the
        // rounding term 2^(S-1), S = 31 + shift >= 33, is a multiple of 2^32, so only the high word of the 64-bit
        // product matters: floor((t + 2^(S-1)) / 2^S) = (hi(t) + 2^(shift-2)) >> (shift-1) exactly, because the low
        // word adds a fraction < 1 to an integer that is then floored by at least one more bit.
        // (out-of-range shifts are detected on the way; the chunk is then redone by the general formula)
        uint32_t in_range = 1;
        const int32_t lo = p.relu ? 0 : -128;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            const int4 b = __ldg(reinterpret_cast<const int4*>(p.bias_i32 + c0 + j));
            const int4 m = __ldg(reinterpret_cast<const int4*>(p.multiplier + c0 + j));
            const int4 t = __ldg(reinterpret_cast<const int4*>(p.shift + c0 + j));
            const int32_t bb[4] = {b.x, b.y, b.z, b.w};
            const int32_t mm[4] = {m.x, m.y, m.z, m.w};
            const int32_t ss[4] = {t.x, t.y, t.z, t.w};
            uint32_t rr[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                in_range &= (uint32_t)((uint32_t)(ss[k] - 2) <= 29u);
                const int32_t acc = (int32_t)((uint32_t)v[j + k] + (uint32_t)bb[k]);
                int32_t r = (__mulhi(acc, mm[k]) + (int32_t)(1u << ((ss[k] - 2) & 31))) >> ((ss[k] - 1) & 31);
                r = r < lo ? lo : r;
                r = r > 127 ? 127 : r;
                rr[k] = (uint32_t)r;
            }
            qw[j >> 2] = __byte_perm(__byte_perm(rr[0], rr[1], 0x0040), __byte_perm(rr[2], rr[3], 0x0040), 0x5410);
        }
        done = in_range != 0;
    }
    if (!done) {
#pragma unroll
        for (int j = 0; j < 8; ++j) qw[j] = 0;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const int c = c0 + j;
            if (j < nch) {
                const int32_t acc = (int32_t)((uint32_t)v[j] + (uint32_t)__ldg(p.bias_i32 + c));
                const int8_t r = requantize_s8(acc, __ldg(p.multiplier + c), __ldg(p.shift + c), p.relu);
                qw[j >> 2] |= (uint32_t)(uint8_t)r << (8 * (j & 3));
            }
        }
    }
}

// Epilogue for one 32-column chunk held by one thread (= one output pixel, 32 consecutive channels).
template <int kOutMode>
__device__ __forceinline__ void epilogue_chunk(const TcParams& p, const uint32_t (&v)[32], int c0, bool valid, int n,
                                               int oh, int ow) {
    if (!valid || c0 >= p.Cout) return;
    const int nch = (p.Cout - c0) < 32 ? (p.Cout - c0) : 32;
    const size_t pix = ((size_t)n * p.OH + oh) * p.OW + ow;

    if constexpr (kOutMode == kOutNHWC_S8 || kOutMode == kOutNCHW_S8) {
        uint32_t qw[8];  // the chunk's 32 int8 results, four per word (bytes in channel order)
        requant_chunk(p, v, c0, nch, qw);
        int8_t* out = static_cast<int8_t*>(p.out);
        if constexpr (kOutMode == kOutNHWC_S8) {
            int8_t* dst = out + pix * p.Cout + c0;
            if (nch == 32 && (p.Cout & 15) == 0 && p.vec_ok) {
                reinterpret_cast<uint4*>(dst)[0] = make_uint4(qw[0], qw[1], qw[2], qw[3]);
                reinterpret_cast<uint4*>(dst)[1] = make_uint4(qw[4], qw[5], qw[6], qw[7]);
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (j < nch) dst[j] = (int8_t)(qw[j >> 2] >> (8 * (j & 3)));
            }
        } else {
            const size_t plane = (size_t)p.OH * p.OW;
            int8_t* dst = out + ((size_t)n * p.Cout + c0) * plane + (size_t)oh * p.OW + ow;
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < nch) dst[(size_t)j * plane] = (int8_t)(qw[j >> 2] >> (8 * (j & 3)));
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


// ---- coalesced variant of the hot-path epilogue --------------------------------------------------
// A thread owns one pixel's 32 channels (64 bytes); pixels of consecutive threads are Cout*2 bytes apart,
// so a warp-wide 16-byte store of thread-owned data touches 32 different lines with 16 bytes each. The
// request rate of such stores (and of the matching residual loads) is what bounds the epilogue. Here the
// chunk passes through a per-warp staging tile in shared memory (32 rows x 64 B): global accesses are issued
// "transposed" -- four neighbouring threads cover the 64 contiguous bytes of ONE pixel, a warp instruction
// covers 8 pixels -- which divides the number of memory requests by four and writes whole 32-byte sectors.
constexpr int kStageTileBytes = 32 * 64;  // 32-row staging tile (a 16-row tile is half of it)

// byte offset of 16-byte piece `piece` (0..3) of row `row` (0..31) inside a staging tile; the XOR keeps both
// the row-owner accesses and the transposed accesses free of bank conflicts
__device__ __forceinline__ uint32_t stage_tile_off(int row, int piece) {
    return (uint32_t)(row * 64 + ((piece ^ ((row >> 1) & 3)) << 4));
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, const uint4& v) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}

// For the transposed accesses thread `lane` handles, in step j (0..3), piece (lane & 3) of row 8*j + (lane >> 2):
// it needs those rows' pixel offsets and validity, which their owner threads hold.
struct RowMap {
    size_t pix[4];
    uint32_t valid;  // bit j: row 8*j + (lane >> 2) is a real output pixel
};
__device__ __forceinline__ RowMap make_row_map(size_t pix, bool valid, int lane) {
    RowMap m;
    m.valid = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int src = 8 * j + (lane >> 2);
        m.pix[j] = (size_t)__shfl_sync(0xffffffffu, (unsigned long long)pix, src);
        m.valid |= (uint32_t)__shfl_sync(0xffffffffu, valid ? 1 : 0, src) << j;
    }
    return m;
}
// What one output tensor's epilogue needs (a kernel with two outputs has two of these).
struct EpiParams {
    const float* bias;     // fp32, may be null
    const void* residual;  // bf16 NHWC like the output, may be null
    void* out;             // bf16 NHWC
    int Cout;
    int relu;
};
// Residual pieces in the transposed arrangement (issued by the caller before it waits for the accumulator).
__device__ __forceinline__ void residual_fetch_rows(const EpiParams& p, const RowMap& m, int c0, int lane, uint4 (&res)[4]) {
    const __nv_bfloat16* base = static_cast<const __nv_bfloat16*>(p.residual) + c0 + (lane & 3) * 8;
#pragma unroll
    for (int j = 0; j < 4; ++j)
        res[j] = ((m.valid >> j) & 1u) ? __ldg(reinterpret_cast<const uint4*>(base + m.pix[j] * p.Cout)) : make_uint4(0, 0, 0, 0);
}
// Residual-free chunk into the warp's store box: 32 rows x 128 bytes (64 channels), SWIZZLE_128B, 1024-byte aligned
// (16-byte piece j of row r sits at piece j ^ (r & 7)). `piece0` = 0 for the first 32 channels of the box, 4 for the
// second. The caller fences and issues the TMA store once both halves are in place.
__device__ __forceinline__ void epilogue_box_bf16(const EpiParams& p, const uint32_t (&v)[32], int c0, uint32_t box, int piece0,
                                                  int lane) {
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
    if (p.relu) {
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = f[j] > 0.0f ? f[j] : 0.0f;
    }
    const uint32_t row = box + (uint32_t)lane * 128u;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        uint4 o;
        o.x = pack_bf16(f[g * 8 + 0], f[g * 8 + 1]);
        o.y = pack_bf16(f[g * 8 + 2], f[g * 8 + 3]);
        o.z = pack_bf16(f[g * 8 + 4], f[g * 8 + 5]);
        o.w = pack_bf16(f[g * 8 + 6], f[g * 8 + 7]);
        st_shared_v4(row + ((uint32_t)((piece0 + g) ^ (lane & 7)) << 4), o);
    }
}

// Whole warp, converged. `tile` = shared-memory address of this warp's staging tile of kPassRows x 64 bytes.
// kPassRows = 32: the warp's 32 rows pass through the tile at once; 16: in two halves (for kernels that can
// spare only 1 KiB of shared memory per epilogue warp).
template <int kPassRows>
__device__ __forceinline__ void epilogue_coalesced_bf16(const EpiParams& p, const uint32_t (&v)[32], int c0, uint32_t tile, int lane,
                                                        const RowMap& m, const uint4 (&res)[4], bool has_res) {
    static_assert(kPassRows == 32 || kPassRows == 16, "staging tile of 32 or 16 rows");
    constexpr int kPasses = 32 / kPassRows;
    constexpr int kSteps = 4 / kPasses;  // transposed steps (8 rows each) per pass
    const int my_pass = lane / kPassRows;
    const int my_row = lane % kPassRows;
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
        for (int h = 0; h < kPasses; ++h) {
#pragma unroll
            for (int js = 0; js < kSteps; ++js)
                st_shared_v4(tile + stage_tile_off(8 * js + (lane >> 2), lane & 3), res[h * kSteps + js]);
            __syncwarp();
            if (kPasses == 1 || my_pass == h) {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const uint4 r = ld_shared_v4(tile + stage_tile_off(my_row, g));
                    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        f[g * 8 + 2 * k] = __fadd_rn(f[g * 8 + 2 * k], bf16_lo(w[k]));
                        f[g * 8 + 2 * k + 1] = __fadd_rn(f[g * 8 + 2 * k + 1], bf16_hi(w[k]));
                    }
                }
            }
            // With one pass every thread next writes the row it has just read; with two, rows are shared
            // between the halves of the warp, so the tile must be quiet before it is written again.
            if (kPasses > 1) __syncwarp();
        }
    }
    if (p.relu) {
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = f[j] > 0.0f ? f[j] : 0.0f;
    }
    uint4 o[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        o[g].x = pack_bf16(f[g * 8 + 0], f[g * 8 + 1]);
        o[g].y = pack_bf16(f[g * 8 + 2], f[g * 8 + 3]);
        o[g].z = pack_bf16(f[g * 8 + 4], f[g * 8 + 5]);
        o[g].w = pack_bf16(f[g * 8 + 6], f[g * 8 + 7]);
    }
    __nv_bfloat16* base = static_cast<__nv_bfloat16*>(p.out) + c0 + (lane & 3) * 8;
#pragma unroll
    for (int h = 0; h < kPasses; ++h) {
        if (kPasses == 1 || my_pass == h) {
#pragma unroll
            for (int g = 0; g < 4; ++g) st_shared_v4(tile + stage_tile_off(my_row, g), o[g]);
        }
        __syncwarp();
#pragma unroll
        for (int js = 0; js < kSteps; ++js) {
            const int j = h * kSteps + js;
            const uint4 q = ld_shared_v4(tile + stage_tile_off(8 * js + (lane >> 2), lane & 3));
            if ((m.valid >> j) & 1u) *reinterpret_cast<uint4*>(base + m.pix[j] * p.Cout) = q;
        }
        __syncwarp();  // the tile may be overwritten (next pass / next chunk)
    }
}

}  // namespace kxc_b200

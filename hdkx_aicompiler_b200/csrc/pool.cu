// Pooling operators on NCHW fp32: nn_max_pool2d, nn_avg_pool2d, nn_global_avg_pool2d and the fused
// chain max_pool2d -> add(residual) -> relu. All HBM-bound; all bit-exact against the reference:
//
//   max : m = -inf; for rh, rw: v = inb ? x : -1e30f; m = (m > v) ? m : v      include/te/topi/nn.h:161-229
//         (explicit compare-select in rh -> rw order, not fmaxf: NaN handling is order dependent)
//   avg : s = 0; for rh, rw: s = s + (inb ? x : 0); out = s / (float)(KH*KW)    include/te/topi/nn.h:231-257
//   gap : s = 0; for h, w: s = s + x; out = s / (float)(H*W)                    include/te/topi/nn.h:260-287
//         (sequential per plane; planes are staged through shared memory so HBM reads stay coalesced)
#include "common.cuh"

#include <cmath>

namespace kxc_b200 {
namespace {

constexpr int kThreads = 256;

struct PoolDims {
    int64_t planes;  // N*C
    int H, W, OH, OW;
    int KH, KW, SH, SW, PT, PL;
};

__device__ __forceinline__ float sel_max(float m, float v) { return (m > v) ? m : v; }
__device__ __forceinline__ float relu1(float v) { return v > 0.0f ? v : 0.0f; }

// ---- generic path: any window/stride/padding, one output per thread-iteration -----------------
template <bool kMax, bool kAddRelu>
__global__ void __launch_bounds__(kThreads) pool_generic_kernel(const float* __restrict__ x,
                                                                const float* __restrict__ res,
                                                                float* __restrict__ out, PoolDims d) {
    const int64_t total = d.planes * d.OH * d.OW;
    const float pad_value = -1e30f;
    const float div = (float)(d.KH * d.KW);
    for (int64_t lin = (int64_t)blockIdx.x * kThreads + threadIdx.x; lin < total; lin += (int64_t)gridDim.x * kThreads) {
        const int ow = (int)(lin % d.OW);
        const int64_t t = lin / d.OW;
        const int oh = (int)(t % d.OH);
        const int64_t plane = t / d.OH;
        const float* xp = x + plane * d.H * d.W;
        float acc = kMax ? -INFINITY : 0.0f;
        for (int rh = 0; rh < d.KH; ++rh) {
            const int ih = oh * d.SH + rh - d.PT;
            for (int rw = 0; rw < d.KW; ++rw) {
                const int iw = ow * d.SW + rw - d.PL;
                const bool inb = (ih >= 0) && (ih < d.H) && (iw >= 0) && (iw < d.W);
                if (kMax) {
                    const float v = inb ? __ldg(xp + (int64_t)ih * d.W + iw) : pad_value;
                    acc = sel_max(acc, v);
                } else {
                    const float v = inb ? __ldg(xp + (int64_t)ih * d.W + iw) : 0.0f;
                    acc = __fadd_rn(acc, v);
                }
            }
        }
        float r = kMax ? acc : __fdiv_rn(acc, div);
        if (kAddRelu) r = relu1(__fadd_rn(r, __ldg(res + lin)));
        out[lin] = r;
    }
}

// ---- fast path: 3x3 window, stride 2, padding 1 (the ResNet stem pool), W % 8 == 0, H even -----
// A thread produces a 2 (rows) x 4 (cols) block of outputs from 5 input rows x 9 input columns:
// two aligned 16-byte loads plus one scalar (the left neighbour) per row. Consecutive threads walk
// consecutive column groups, so every input row is read in contiguous 32-byte pieces and every
// output row is written as contiguous 16-byte vectors.
template <bool kAddRelu>
__global__ void __launch_bounds__(kThreads) maxpool_3x3s2p1_kernel(const float* __restrict__ x,
                                                                   const float* __restrict__ res,
                                                                   float* __restrict__ out, int64_t planes, int H, int W,
                                                                   int OH, int OW) {
    const int groups = OW >> 2;        // 4 outputs per group
    const int row_pairs = OH >> 1;     // OH is even when this kernel is chosen
    const int64_t total = planes * row_pairs * groups;
    const float pad_value = -1e30f;
    for (int64_t lin = (int64_t)blockIdx.x * kThreads + threadIdx.x; lin < total; lin += (int64_t)gridDim.x * kThreads) {
        const int g = (int)(lin % groups);
        const int64_t t = lin / groups;
        const int rp = (int)(t % row_pairs);
        const int64_t plane = t / row_pairs;
        const int ow0 = g << 2;
        const int oh0 = rp << 1;
        const int iw0 = ow0 * 2;  // multiple of 8 -> 32-byte aligned in an aligned row
        const float* xp = x + plane * (int64_t)H * W;

        float r[5][9];
#pragma unroll
        for (int j = 0; j < 5; ++j) {
            const int ih = oh0 * 2 - 1 + j;
            if (ih >= 0 && ih < H) {
                const float* row = xp + (int64_t)ih * W;
                const float4 a = __ldg(reinterpret_cast<const float4*>(row + iw0));
                const float4 b = __ldg(reinterpret_cast<const float4*>(row + iw0 + 4));
                r[j][0] = (iw0 > 0) ? __ldg(row + iw0 - 1) : pad_value;
                r[j][1] = a.x; r[j][2] = a.y; r[j][3] = a.z; r[j][4] = a.w;
                r[j][5] = b.x; r[j][6] = b.y; r[j][7] = b.z; r[j][8] = b.w;
            } else {
#pragma unroll
                for (int c = 0; c < 9; ++c) r[j][c] = pad_value;
            }
        }
#pragma unroll
        for (int orow = 0; orow < 2; ++orow) {
            float o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float m = -INFINITY;
#pragma unroll
                for (int rh = 0; rh < 3; ++rh)
#pragma unroll
                    for (int rw = 0; rw < 3; ++rw) m = sel_max(m, r[orow * 2 + rh][j * 2 + rw]);
                o[j] = m;
            }
            const int64_t off = (plane * OH + oh0 + orow) * (int64_t)OW + ow0;
            if (kAddRelu) {
                const float4 rv = __ldcs(reinterpret_cast<const float4*>(res + off));
                o[0] = relu1(__fadd_rn(o[0], rv.x));
                o[1] = relu1(__fadd_rn(o[1], rv.y));
                o[2] = relu1(__fadd_rn(o[2], rv.z));
                o[3] = relu1(__fadd_rn(o[3], rv.w));
            }
            __stcs(reinterpret_cast<float4*>(out + off), make_float4(o[0], o[1], o[2], o[3]));
        }
    }
}

// ---- global average pool: coalesced staging, sequential per-plane sum --------------------------
// kLinear: the CTA's planes are copied into shared memory exactly as they lie in global memory, 16 bytes per access
// (odd plane sizes only: the per-thread sequential walk with an odd stride hits distinct banks). Otherwise planes are
// padded to an odd pitch and the (plane, offset) pair of each element is advanced without divisions.
template <bool kLinear>
__global__ void __launch_bounds__(128) gap_staged_kernel(const float* __restrict__ x, float* __restrict__ out,
                                                         int64_t planes, int HW, int planes_per_cta, int pitch) {
    extern __shared__ __align__(16) float tile[];
    const float div = (float)HW;
    for (int64_t p0 = (int64_t)blockIdx.x * planes_per_cta; p0 < planes; p0 += (int64_t)gridDim.x * planes_per_cta) {
        const int np = (int)((planes - p0 < planes_per_cta) ? (planes - p0) : planes_per_cta);
        const float* src = x + p0 * HW;
        const int count = np * HW;
        if (kLinear) {
            const float4* src4 = reinterpret_cast<const float4*>(src);
            const int n4 = count >> 2;
            // asynchronous 16-byte copies straight into shared memory: all of a thread's copies are in flight at once
            // and none of them holds a register
            const uint32_t tile_addr = (uint32_t)__cvta_generic_to_shared(tile);
            for (int i = threadIdx.x; i < n4; i += 128)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(tile_addr + (uint32_t)i * 16u), "l"(src4 + i) : "memory");
            asm volatile("cp.async.commit_group;" ::: "memory");
            for (int j = (n4 << 2) + threadIdx.x; j < count; j += 128) tile[j] = __ldcs(src + j);
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        } else {
            int p = threadIdx.x / HW, r = threadIdx.x - p * HW;
            const int dp = 128 / HW, dr = 128 - dp * HW;
            for (int i = threadIdx.x; i < count; i += 128) {
                tile[p * pitch + r] = __ldcs(src + i);
                p += dp;
                r += dr;
                if (r >= HW) {
                    r -= HW;
                    ++p;
                }
            }
        }
        __syncthreads();
        for (int p = threadIdx.x; p < np; p += blockDim.x) {
            const float* row = tile + p * pitch;
            float s = 0.0f;
#pragma unroll 7
            for (int i = 0; i < HW; ++i) s = __fadd_rn(s, row[i]);  // the unrolled loads run ahead of the add chain
            out[p0 + p] = __fdiv_rn(s, div);
        }
        __syncthreads();
    }
}

// Planes too large to stage: each thread still walks its plane sequentially (exact), uncoalesced.
__global__ void gap_direct_kernel(const float* __restrict__ x, float* __restrict__ out, int64_t planes, int64_t HW) {
    const float div = (float)HW;
    for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < planes; p += (int64_t)gridDim.x * blockDim.x) {
        const float* row = x + p * HW;
        float s = 0.0f;
        for (int64_t i = 0; i < HW; ++i) s = __fadd_rn(s, __ldg(row + i));
        out[p] = __fdiv_rn(s, div);
    }
}

int grid_for(int64_t items, int threads, int blocks_per_sm) {
    int64_t blocks = (items + threads - 1) / threads;
    const int64_t cap = (int64_t)kNumSMs * blocks_per_sm;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

int32_t validate_pool(const kxc_b200_pool2d_desc* d, const char* name, PoolDims* out) {
    if (!d) return fail(KXC_B200_ERR_INVALID, "%s: null descriptor", name);
    if (d->n < 0 || d->c < 0 || d->h <= 0 || d->w <= 0 || d->kh <= 0 || d->kw <= 0 || d->stride_h <= 0 ||
        d->stride_w <= 0 || d->pad_top < 0 || d->pad_left < 0 || d->pad_bottom < 0 || d->pad_right < 0)
        return fail(KXC_B200_ERR_INVALID, "%s: bad shape/window/stride/padding", name);
    const int64_t OH = pool_out_dim(d->h, d->kh, d->stride_h, d->pad_top, d->pad_bottom, d->ceil_mode != 0);
    const int64_t OW = pool_out_dim(d->w, d->kw, d->stride_w, d->pad_left, d->pad_right, d->ceil_mode != 0);
    if (OH <= 0 || OW <= 0) return fail(KXC_B200_ERR_INVALID, "%s: empty output (%lld x %lld)", name, (long long)OH, (long long)OW);
    out->planes = (int64_t)d->n * d->c;
    out->H = d->h; out->W = d->w; out->OH = (int)OH; out->OW = (int)OW;
    out->KH = d->kh; out->KW = d->kw; out->SH = d->stride_h; out->SW = d->stride_w;
    out->PT = d->pad_top; out->PL = d->pad_left;
    return KXC_B200_OK;
}

template <bool kAddRelu>
int32_t launch_max_pool(const float* x, const float* res, float* out, const kxc_b200_pool2d_desc* d, const PoolDims& pd,
                        cudaStream_t s, const char* name) {
    if (pd.planes == 0) return KXC_B200_OK;
    const bool fast = d->kh == 3 && d->kw == 3 && d->stride_h == 2 && d->stride_w == 2 && d->pad_top == 1 &&
                      d->pad_left == 1 && d->pad_bottom == 1 && d->pad_right == 1 && (d->w % 8 == 0) && (d->h % 4 == 0) &&
                      aligned16(x) && aligned16(out) && (!kAddRelu || aligned16(res));
    if (fast) {
        const int64_t items = pd.planes * (pd.OH / 2) * (pd.OW / 4);
        // one item per thread (no grid-stride iterations) up to 64 blocks per SM: the hardware block scheduler
        // balances these short kernels at a finer grain than a persistent loop would
        maxpool_3x3s2p1_kernel<kAddRelu><<<grid_for(items, kThreads, 64), kThreads, 0, s>>>(x, res, out, pd.planes, pd.H,
                                                                                           pd.W, pd.OH, pd.OW);
    } else {
        const int64_t items = pd.planes * pd.OH * pd.OW;
        pool_generic_kernel<true, kAddRelu><<<grid_for(items, kThreads, 8), kThreads, 0, s>>>(x, res, out, pd);
    }
    return check_launch(name);
}

}  // namespace
}  // namespace kxc_b200

using namespace kxc_b200;

extern "C" int32_t kxc_b200_nn_max_pool2d(void** packed_args, const kxc_b200_pool2d_desc* desc, void* stream) {
    KXC_TRY(require_device());
    PoolDims pd;
    KXC_TRY(validate_pool(desc, "nn_max_pool2d", &pd));
    if (pd.planes == 0) return KXC_B200_OK;
    if (!packed_args || !packed_args[0] || !packed_args[1]) return fail(KXC_B200_ERR_INVALID, "nn_max_pool2d: null tensor pointer");
    return launch_max_pool<false>(static_cast<const float*>(packed_args[0]), nullptr, static_cast<float*>(packed_args[1]),
                                  desc, pd, static_cast<cudaStream_t>(stream), "nn_max_pool2d");
}

extern "C" int32_t kxc_b200_max_pool2d_add_relu(void** packed_args, const kxc_b200_pool2d_desc* desc, void* stream) {
    KXC_TRY(require_device());
    PoolDims pd;
    KXC_TRY(validate_pool(desc, "max_pool2d_add_relu", &pd));
    if (pd.planes == 0) return KXC_B200_OK;
    if (!packed_args || !packed_args[0] || !packed_args[1] || !packed_args[2])
        return fail(KXC_B200_ERR_INVALID, "max_pool2d_add_relu: null tensor pointer");
    return launch_max_pool<true>(static_cast<const float*>(packed_args[0]), static_cast<const float*>(packed_args[1]),
                                 static_cast<float*>(packed_args[2]), desc, pd, static_cast<cudaStream_t>(stream),
                                 "max_pool2d_add_relu");
}

extern "C" int32_t kxc_b200_nn_avg_pool2d(void** packed_args, const kxc_b200_pool2d_desc* desc, void* stream) {
    KXC_TRY(require_device());
    PoolDims pd;
    KXC_TRY(validate_pool(desc, "nn_avg_pool2d", &pd));
    if (pd.planes == 0) return KXC_B200_OK;
    if (!packed_args || !packed_args[0] || !packed_args[1]) return fail(KXC_B200_ERR_INVALID, "nn_avg_pool2d: null tensor pointer");
    if (pd.planes == 0) return KXC_B200_OK;
    const int64_t items = pd.planes * pd.OH * pd.OW;
    pool_generic_kernel<false, false><<<grid_for(items, kThreads, 8), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const float*>(packed_args[0]), nullptr, static_cast<float*>(packed_args[1]), pd);
    return check_launch("nn_avg_pool2d");
}

extern "C" int32_t kxc_b200_nn_global_avg_pool2d(void** packed_args, int32_t n, int32_t c, int32_t h, int32_t w,
                                                 void* stream) {
    KXC_TRY(require_device());
    if (n < 0 || c < 0 || h <= 0 || w <= 0) return fail(KXC_B200_ERR_INVALID, "nn_global_avg_pool2d: bad shape");
    const int64_t planes = (int64_t)n * c;
    if (planes == 0) return KXC_B200_OK;
    if (!packed_args || !packed_args[0] || !packed_args[1])
        return fail(KXC_B200_ERR_INVALID, "nn_global_avg_pool2d: null tensor pointer");
    const int64_t HW = (int64_t)h * w;
    const float* x = static_cast<const float*>(packed_args[0]);
    float* out = static_cast<float*>(packed_args[1]);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    constexpr int kSmemBudget = 40 * 1024;
    const bool linear = (HW & 1) && aligned16(x);
    const int64_t pitch = linear ? HW : (HW | 1);  // odd pitch: the per-thread sequential walk hits distinct banks
    if (pitch * 4 * 8 <= kSmemBudget) {
        int per_cta = (int)(kSmemBudget / (pitch * 4));
        if (per_cta > 128) per_cta = 128;
        per_cta &= ~3;  // every CTA's first plane then starts on a 16-byte boundary
        const int64_t ctas = (planes + per_cta - 1) / per_cta;
        // one CTA per group of planes (no grid-stride loop unless the count exceeds the grid limit): the hardware
        // hands out CTAs as SMs free up, which balances better than a fixed 3-or-4 iterations per resident CTA
        const int grid = (int)(ctas < 0x7fffffff ? ctas : 0x7fffffff);
        if (linear)
            gap_staged_kernel<true><<<grid, 128, (size_t)per_cta * pitch * 4, s>>>(x, out, planes, (int)HW, per_cta, (int)pitch);
        else
            gap_staged_kernel<false><<<grid, 128, (size_t)per_cta * pitch * 4, s>>>(x, out, planes, (int)HW, per_cta, (int)pitch);
    } else {
        gap_direct_kernel<<<grid_for(planes, 128, 8), 128, 0, s>>>(x, out, planes, HW);
    }
    return check_launch("nn_global_avg_pool2d");
}

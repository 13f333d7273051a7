// softmax and reduce_mean on fp32 tensors in the reference's row-major layout.
//
//   softmax     e = exp(x); s = 0; s = s + e along the axis; out = e / s — no subtraction of the maximum
//               (src/relay/op/nn/softmax.cc:44-70). The reference's reduction indexes the wrong elements when a
//               kept dimension FOLLOWS the reduced one and keepdims is set (include/te/topi/reduction.h:47-58 advances
//               its output-index counter only for kept dimensions), which is the case for every softmax axis but the
//               last: only the last axis is accepted. exp() comes from the device's math library, so results agree
//               with the CPU's to a few ulp, not bit for bit; the sum is a block reduction.
//   reduce_mean s = 0; s = s + x with the reduced axes as nested loops in ascending order; out = s / (float)count
//               (src/relay/op/tensor/reduce.cc:81-99). Bit-exact: one thread walks one output's elements in that
//               order. Reduced trailing axes take the staged, coalesced kernel of nn_global_avg_pool2d. With keepdims
//               the same reference defect applies unless the reduced axes are the trailing ones, so keepdims = 1 is
//               accepted for trailing axes only.
#include "common.cuh"

namespace kxc_b200 {
namespace {

constexpr int kSoftmaxThreads = 128;

__global__ void __launch_bounds__(kSoftmaxThreads) softmax_rows_kernel(const float* __restrict__ x, float* __restrict__ out,
                                                                     int64_t rows, int len) {
    __shared__ float warp_sum[kSoftmaxThreads / 32];
    __shared__ float total;
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const float* xp = x + r * len;
        float* op = out + r * len;
        float s = 0.0f;
        for (int i = threadIdx.x; i < len; i += kSoftmaxThreads) s = __fadd_rn(s, expf(xp[i]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, o));
        if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = s;
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = 0.0f;
            for (int w = 0; w < kSoftmaxThreads / 32; ++w) t = __fadd_rn(t, warp_sum[w]);
            total = t;
        }
        __syncthreads();
        const float denom = total;
        for (int i = threadIdx.x; i < len; i += kSoftmaxThreads) op[i] = __fdiv_rn(expf(xp[i]), denom);
        __syncthreads();
    }
}

// Rows of at most kPer * 128 elements: every thread keeps its exponentials in registers, so the row is read once and
// expf runs once per element. Same summation order as softmax_rows_kernel (thread-strided partial sums, warp shuffles,
// warps in order), hence the same bits.
template <int kPer>
__global__ void __launch_bounds__(kSoftmaxThreads) softmax_rows_reg_kernel(const float* __restrict__ x, float* __restrict__ out,
                                                                         int64_t rows, int len) {
    __shared__ float warp_sum[2][kSoftmaxThreads / 32];
    int phase = 0;
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x, phase ^= 1) {
        const float* xp = x + r * len;
        float* op = out + r * len;
        float e[kPer];
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
            const int i = threadIdx.x + k * kSoftmaxThreads;
            e[k] = i < len ? __ldcs(xp + i) : 0.0f;
        }
        float s = 0.0f;
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
            const int i = threadIdx.x + k * kSoftmaxThreads;
            if (i < len) {
                e[k] = expf(e[k]);
                s = __fadd_rn(s, e[k]);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, o));
        if ((threadIdx.x & 31) == 0) warp_sum[phase][threadIdx.x >> 5] = s;
        __syncthreads();  // the buffer alternates between rows, so one barrier per row is enough
        float denom = 0.0f;
#pragma unroll
        for (int w = 0; w < kSoftmaxThreads / 32; ++w) denom = __fadd_rn(denom, warp_sum[phase][w]);
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
            const int i = threadIdx.x + k * kSoftmaxThreads;
            if (i < len) __stcs(op + i, __fdiv_rn(e[k], denom));
        }
    }
}

struct ReduceDims {
    int nk, nr;               // kept / reduced dimensions
    int64_t kshape[6], kstride[6];
    int64_t rshape[6], rstride[6];
    int64_t count, nout;
};

__global__ void reduce_mean_kernel(const float* __restrict__ x, float* __restrict__ out, ReduceDims d) {
    const float div = (float)d.count;
    for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < d.nout; o += (int64_t)gridDim.x * blockDim.x) {
        int64_t rem = o, base = 0;
        for (int j = d.nk - 1; j >= 0; --j) {
            base += (rem % d.kshape[j]) * d.kstride[j];
            rem /= d.kshape[j];
        }
        float s = 0.0f;
        int64_t idx[6] = {0, 0, 0, 0, 0, 0};
        int64_t off = base;
        for (int64_t r = 0; r < d.count; ++r) {
            s = __fadd_rn(s, __ldg(x + off));
            // next element in the order of the reference's loop nest: the last reduced axis runs fastest
            for (int j = d.nr - 1; j >= 0; --j) {
                off += d.rstride[j];
                if (++idx[j] < d.rshape[j]) break;
                off -= idx[j] * d.rstride[j];
                idx[j] = 0;
            }
        }
        out[o] = __fdiv_rn(s, div);
    }
}

}  // namespace
}  // namespace kxc_b200

using namespace kxc_b200;

extern "C" int32_t kxc_b200_softmax(void** packed_args, const kxc_b200_softmax_desc* desc, void* stream) {
    KXC_TRY(require_device());
    if (!packed_args || !desc) return fail(KXC_B200_ERR_INVALID, "softmax: bad arguments");
    if (desc->rank < 1 || desc->rank > 6) return fail(KXC_B200_ERR_INVALID, "softmax: rank must be in [1,6]");
    int axis = desc->axis < 0 ? desc->axis + desc->rank : desc->axis;
    if (axis < 0 || axis >= desc->rank) return fail(KXC_B200_ERR_INVALID, "softmax: axis %d out of range for rank %d", desc->axis, desc->rank);
    if (axis != desc->rank - 1)
        return fail(KXC_B200_ERR_UNSUPPORTED, "softmax: only the last axis is supported (the reference's reduction over an inner axis "
                                             "reads the wrong elements)");
    int64_t rows = 1;
    for (int i = 0; i < desc->rank - 1; ++i) {
        if (desc->shape[i] < 0) return fail(KXC_B200_ERR_INVALID, "softmax: negative extent");
        rows *= desc->shape[i];
    }
    const int64_t len = desc->shape[axis];
    if (len < 0 || len > 0x7fffffff) return fail(KXC_B200_ERR_INVALID, "softmax: bad axis length");
    if (rows == 0 || len == 0) return KXC_B200_OK;
    if (!packed_args[0] || !packed_args[1]) return fail(KXC_B200_ERR_INVALID, "softmax: null tensor pointer");
    const int grid = (int)(rows < (int64_t)kNumSMs * 16 ? rows : (int64_t)kNumSMs * 16);
    const float* xin = static_cast<const float*>(packed_args[0]);
    float* yout = static_cast<float*>(packed_args[1]);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (len <= 4 * kSoftmaxThreads)
        softmax_rows_reg_kernel<4><<<grid, kSoftmaxThreads, 0, s>>>(xin, yout, rows, (int)len);
    else if (len <= 8 * kSoftmaxThreads)
        softmax_rows_reg_kernel<8><<<grid, kSoftmaxThreads, 0, s>>>(xin, yout, rows, (int)len);
    else if (len <= 16 * kSoftmaxThreads)
        softmax_rows_reg_kernel<16><<<grid, kSoftmaxThreads, 0, s>>>(xin, yout, rows, (int)len);
    else
        softmax_rows_kernel<<<grid, kSoftmaxThreads, 0, s>>>(xin, yout, rows, (int)len);
    return check_launch("softmax");
}

extern "C" int32_t kxc_b200_reduce_mean(void** packed_args, const kxc_b200_reduce_desc* desc, void* stream) {
    KXC_TRY(require_device());
    if (!packed_args || !desc) return fail(KXC_B200_ERR_INVALID, "reduce_mean: bad arguments");
    if (desc->rank < 1 || desc->rank > 6) return fail(KXC_B200_ERR_INVALID, "reduce_mean: rank must be in [1,6]");
    if (desc->num_axes < 1 || desc->num_axes > desc->rank) return fail(KXC_B200_ERR_INVALID, "reduce_mean: bad number of axes");
    bool reduced[6] = {false, false, false, false, false, false};
    for (int i = 0; i < desc->num_axes; ++i) {
        const int a = desc->axes[i] < 0 ? desc->axes[i] + desc->rank : desc->axes[i];
        if (a < 0 || a >= desc->rank || reduced[a]) return fail(KXC_B200_ERR_INVALID, "reduce_mean: bad axis %d", desc->axes[i]);
        reduced[a] = true;
    }
    int first_reduced = desc->rank;
    for (int i = desc->rank - 1; i >= 0 && reduced[i]; --i) first_reduced = i;
    bool trailing = true;  // all reduced axes at the end
    for (int i = 0; i < first_reduced; ++i) trailing = trailing && !reduced[i];
    if (desc->keepdims && !trailing)
        return fail(KXC_B200_ERR_UNSUPPORTED, "reduce_mean: keepdims with a kept dimension after a reduced one is not supported (the "
                                             "reference's reduction reads the wrong elements there)");
    ReduceDims d{};
    int64_t stride[6];
    int64_t st = 1;
    for (int i = desc->rank - 1; i >= 0; --i) {
        if (desc->shape[i] < 0) return fail(KXC_B200_ERR_INVALID, "reduce_mean: negative extent");
        stride[i] = st;
        st *= desc->shape[i];
    }
    d.count = 1;
    d.nout = 1;
    for (int i = 0; i < desc->rank; ++i) {
        if (reduced[i]) {
            d.rshape[d.nr] = desc->shape[i];
            d.rstride[d.nr++] = stride[i];
            d.count *= desc->shape[i];
        } else {
            d.kshape[d.nk] = desc->shape[i];
            d.kstride[d.nk++] = stride[i];
            d.nout *= desc->shape[i];
        }
    }
    if (d.nout == 0) return KXC_B200_OK;
    if (d.count == 0) return fail(KXC_B200_ERR_INVALID, "reduce_mean: empty reduction");
    if (!packed_args[0] || !packed_args[1]) return fail(KXC_B200_ERR_INVALID, "reduce_mean: null tensor pointer");
    if (trailing && d.nout <= 0x7fffffff && d.count <= 0x7fffffff) {
        // [planes, count] with contiguous planes: the global-average kernel (sequential per plane, coalesced staging)
        return kxc_b200_nn_global_avg_pool2d(packed_args, 1, (int32_t)d.nout, 1, (int32_t)d.count, stream);
    }
    const int64_t blocks = (d.nout + 127) / 128;
    const int grid = (int)(blocks < (int64_t)kNumSMs * 16 ? blocks : (int64_t)kNumSMs * 16);
    reduce_mean_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const float*>(packed_args[0]),
                                                                          static_cast<float*>(packed_args[1]), d);
    return check_launch("reduce_mean");
}

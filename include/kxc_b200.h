/* kxc_b200.h — C ABI of libkxc_b200.so: hand-written sm_100a kernels for the operators that the
 * hdkx-aicompiler ("kxc") Relay graphs lower into, callable from the compiler's C++ runtime.
 *
 * Conventions (all taken from the reference so the library drops into its kernel slot):
 *  - Entry points take `void** packed_args`: raw data pointers, inputs first, outputs last — the
 *    packed ABI of `CompiledKernel::operator()` (src/codegen/compiled_kernel.cc:41-55) and of the
 *    generated `int32_t kxc_kernel_main(void** packed_args)` (src/codegen/codegen_llvm.cc:56-63,
 *    parameter order from src/relay/backend/lower.cc:534-565). Pointers are DEVICE pointers
 *    (what `DeviceAPI::AllocDataSpace` returns for a CUDA device, src/base/device/cuda_device_api.cc:89-105).
 *  - Return value: 0 = success, non-zero = error (the caller turns it into
 *    "Kernel <name> returned error code N", compiled_kernel.cc:50-54). Nothing throws across this
 *    boundary; `kxc_b200_last_error()` gives the message for the calling thread.
 *  - Tensors are dense row-major NCHW / OIHW float32 unless stated (src/relay/backend/lower.cc:59-71).
 *  - `stream` is a `cudaStream_t` (the reference keeps it thread-local in DeviceAPI,
 *    cuda_device_api.cc:23,273-298; NULL = the legacy default stream). Launches are asynchronous;
 *    synchronising is the caller's job, like `DeviceAPI::StreamSync`.
 *  - The caller owns every buffer in `packed_args`; the library owns its workspaces and packed weights.
 *  - There is no CPU fallback: without a CUDA device every compute entry point returns an error.
 */
#ifndef KXC_B200_H_
#define KXC_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KXC_B200_ABI_VERSION 1

/* error codes (non-zero = failure) */
enum {
    KXC_B200_OK = 0,
    KXC_B200_ERR_INVALID = 1,      /* bad descriptor, null pointer, shape mismatch            */
    KXC_B200_ERR_UNSUPPORTED = 2,  /* legal for the reference, not implemented by this library */
    KXC_B200_ERR_CUDA = 3,         /* a CUDA runtime/driver call failed                        */
    KXC_B200_ERR_NO_DEVICE = 4,    /* no sm_100 device: there is no CPU fallback               */
    KXC_B200_ERR_DEVICE_WAIT = 5,  /* a bounded device-side wait ran out (status word set)     */
    KXC_B200_ERR_NOMEM = 6
};

/* fused-epilogue flags for conv2d / dense */
enum {
    KXC_B200_BIAS = 1,     /* + bias[o]          (src/relay/op/nn/convolution.cc:72-74)       */
    KXC_B200_RESIDUAL = 2, /* + residual[n,o,h,w] (the `add` that follows in a BasicBlock)     */
    KXC_B200_RELU = 4,     /* x > 0 ? x : 0      (include/te/topi/nn.h:19-30)                 */
    KXC_B200_NHWC = 8      /* kxc_b200_nn_conv2d_s8 only: operands already in the kernel's layout  */
};

/* arithmetic mode of the contraction */
enum {
    KXC_B200_PREC_FP32 = 0, /* CUDA-core fp32, the reference's rc->rh->rw order, separately rounded mul/add: bit-exact */
    KXC_B200_PREC_TF32 = 1, /* tcgen05 kind::tf32, operands rounded to tf32 (RNE), fp32 accumulate in TMEM */
    KXC_B200_PREC_BF16 = 2, /* tcgen05 kind::f16 (bf16), operands rounded to bf16 (RNE), fp32 accumulate   */
    KXC_B200_PREC_SIMT = 3, /* int8 entry point only: force the CUDA-core kernel instead of tcgen05 kind::i8 */
    KXC_B200_PREC_TF32X3 = 4 /* per-op conv / gemm / matmul: operands split into tf32 high and low parts, three tcgen05
                                passes (lo*hi, hi*lo, hi*hi) summed in fp32: fp32-class accuracy on the tensor cores */
};

const char* kxc_b200_last_error(void);
int32_t kxc_b200_abi_version(void);
/* 0 when a device with compute capability 10.x is present and usable, else KXC_B200_ERR_NO_DEVICE. */
int32_t kxc_b200_device_check(void);
/* The tensor-core kernels bound every device-side wait; one that runs out sets a device status word
 * instead of hanging. This call synchronises `stream`, returns that word in *status_out (0 = clean)
 * and clears it; its return value is non-zero when the word was set. The kernels launched by
 * kxc_b200_nn_conv2d_static_scratch report into a word of their own, which this call reads, ORs into the
 * result and clears as well. No reference counterpart: the reference's kernels are synchronous CPU
 * loops (src/codegen/compiled_kernel.cc:41-55). */
int32_t kxc_b200_device_status(void* stream, int32_t* status_out);

/* Self tests of the library's safety plumbing (no reference counterpart).
 * selftest_bounded_wait: launches ONE small kernel whose only thread waits, through the bounded wait every
 *   tensor-core kernel uses, on a barrier nothing ever arrives on. After `limit_ns` (at most 100 ms) the wait
 *   gives up, the kernel sets the device status word to KXC_B200_ERR_DEVICE_WAIT and returns normally;
 *   *gave_up_out = 1. A following kxc_b200_device_status call must report and clear the word. Nothing hangs,
 *   traps or faults: this is the path a protocol error in a real kernel would take.
 * selftest_per_device_once: host only (runs without a GPU): checks the once-per-device bookkeeping that repeats
 *   the shared-memory opt-in of every kernel on each device of a multi-GPU process. Returns 0 when it holds. */
int32_t kxc_b200_selftest_bounded_wait(int64_t limit_ns, void* stream, int32_t* gave_up_out);
int32_t kxc_b200_selftest_per_device_once(void);

/* Threading. Every per-operator entry point of this header is re-entrant: it keeps no mutable state besides
 * thread-safe caches (device check, per-device kernel attributes, the status words) and a per-thread error
 * message, so several host threads may call the same or different entry points at the same time, each on its
 * own stream, as the reference's KernelRunner does (src/runtime/kernel_runner.cc:17-30). The exceptions are
 * spelled out where they apply: kxc_b200_nn_conv2d_static_scratch (one shared workspace) here, and a
 * kxc_b200_plan object in kxc_b200_plan.h (one run in flight per plan). */

/* ---------------------------------------------------------------------------------------------
 * nn_conv2d — replaces the kernel generated from topi::conv2d_nchw (include/te/topi/nn.h:107-158)
 * via Conv2DCompute (src/relay/op/nn/convolution.cc:38-75).
 * packed_args = { data[N,C,H,W], weight[O,C,KH,KW], (bias[O] if BIAS), (residual[N,O,OH,OW] if RESIDUAL),
 *                 out[N,O,OH,OW] }.  Padding is symmetric (padding[0], padding[1]) like the reference;
 * groups must be 1 (the reference ignores groups in compute, src/relay/type_infer.cc:364-368).
 * Epilogue order: acc -> +bias -> +residual -> relu, each a separately rounded fp32 step. */
typedef struct kxc_b200_conv2d_desc {
    int32_t n, c, h, w;
    int32_t o, kh, kw;
    int32_t stride_h, stride_w;
    int32_t pad_h, pad_w;
    int32_t dilation_h, dilation_w;
    int32_t flags;     /* KXC_B200_BIAS | KXC_B200_RESIDUAL | KXC_B200_RELU */
    int32_t precision; /* KXC_B200_PREC_* */
} kxc_b200_conv2d_desc;

int32_t kxc_b200_nn_conv2d(void** packed_args, const kxc_b200_conv2d_desc* desc, void* stream);

/* nn_conv2d on the tensor cores WITHOUT any allocation (no counterpart in the reference, whose kernels
 * malloc their intermediates on every call, src/codegen/codegen_llvm.cc:591-616).
 * Same arguments and results as kxc_b200_nn_conv2d with precision KXC_B200_PREC_BF16 / _TF32, for hosts
 * that cannot call the CUDA allocator at run time (a runtime that owns all device memory through its own
 * pool, a latency-critical loop that may not take allocator locks). The operand workspace is a fixed
 * array inside the library: each GPU that loads the library holds kxc_b200_static_scratch_bytes()
 * (32 MiB) for it until exit. A convolution whose converted activations + packed weights exceed that
 * size is rejected with KXC_B200_ERR_NOMEM. All calls share the array: calls whose GPU work overlaps
 * (different streams) race, so keep them on one stream. The first call on a device resolves the array's
 * address; make it before any stream capture begins. */
int32_t kxc_b200_nn_conv2d_static_scratch(void** packed_args, const kxc_b200_conv2d_desc* desc, void* stream);
int64_t kxc_b200_static_scratch_bytes(void);

/* int8 convolution with int32 accumulate and fixed-point requantize. The reference has no quantized
 * op; accumulators equal its nn_conv2d run on the int8 values widened to int32 (include/te/topi/nn.h:107-158).
 * packed_args = { data int8[N,C,H,W], weight int8[O,C,KH,KW], bias int32[O], multiplier int32[O],
 *                 shift int32[O], out int8[N,O,OH,OW] }.
 * y = sat8( relu?( (acc*M + 2^(30+shift)) >> (31+shift) ) ), 64-bit, arithmetic shift.
 * desc->precision: KXC_B200_PREC_SIMT forces the CUDA-core kernel, anything else takes the tcgen05
 * kind::i8 path (both are integer-exact). desc->flags: BIAS is required, RELU optional.
 * With KXC_B200_NHWC (tensor-core path only) the tensors stay in the kernel's own layout from call to call, as in a
 * quantized pipeline: data int8[N,H,W,C], weight int8[O,KH,KW,C], out int8[N,OH,OW,O], with C a multiple of 32 up to
 * 128 or a multiple of 128, O a multiple of 16 and 16-byte aligned pointers; no conversion kernels run and no
 * workspace is allocated. One exception to the channel rule: a stride-2 first layer with C <= 8, O == 64 and a
 * filter of at most 7 x 8 (an image stem) keeps its raw [N,H,W,C] pixels; the library packs them to 8 bytes each in a
 * workspace and runs its direct stem kernel. The values are those of the reference layout, permuted. */
int32_t kxc_b200_nn_conv2d_s8(void** packed_args, const kxc_b200_conv2d_desc* desc, void* stream);

/* nn_relu — topi::relu (include/te/topi/nn.h:19-30) via ReluCompute (src/relay/op/nn/activation.cc:14-19).
 * packed_args = { x[numel], out[numel] } */
int32_t kxc_b200_nn_relu(void** packed_args, int64_t numel, void* stream);

/* add — topi::add (include/te/topi/broadcast.h:90-109) via AddCompute (src/relay/op/tensor/math.cc:41-47).
 * Right-aligned NumPy broadcast: an input dim of 1 reads index 0. rank <= 6.
 * packed_args = { a, b, out } */
typedef struct kxc_b200_add_desc {
    int32_t rank_a, rank_b;
    int64_t shape_a[6];
    int64_t shape_b[6];
    int32_t relu; /* 0 = plain add; 1 = also apply nn_relu to the sum (fused add -> relu) */
} kxc_b200_add_desc;
int32_t kxc_b200_add(void** packed_args, const kxc_b200_add_desc* desc, void* stream);

/* nn_max_pool2d / nn_avg_pool2d — topi::pool2d (include/te/topi/nn.h:161-257) via MaxPool2DCompute /
 * AvgPool2DCompute (src/relay/op/nn/pooling.cc:50-86). padding = (top, left, bottom, right).
 * packed_args = { x[N,C,H,W], out[N,C,OH,OW] } */
typedef struct kxc_b200_pool2d_desc {
    int32_t n, c, h, w;
    int32_t kh, kw;
    int32_t stride_h, stride_w;
    int32_t pad_top, pad_left, pad_bottom, pad_right;
    int32_t ceil_mode;
} kxc_b200_pool2d_desc;
int32_t kxc_b200_nn_max_pool2d(void** packed_args, const kxc_b200_pool2d_desc* desc, void* stream);
int32_t kxc_b200_nn_avg_pool2d(void** packed_args, const kxc_b200_pool2d_desc* desc, void* stream);

/* Fused memory-bound chain nn_max_pool2d -> add(residual) -> nn_relu in ONE pass over HBM.
 * Same values as the three reference loop nests run back to back (each step is exact).
 * packed_args = { x[N,C,H,W], residual[N,C,OH,OW], out[N,C,OH,OW] } */
int32_t kxc_b200_max_pool2d_add_relu(void** packed_args, const kxc_b200_pool2d_desc* desc, void* stream);

/* softmax — SoftmaxCompute (src/relay/op/nn/softmax.cc:44-70): exp, sum along the axis in index order, divide; no
 * subtraction of the maximum. packed_args = { x, out } of the same shape. Only the last axis is accepted: for any other
 * axis the reference's keepdims reduction (include/te/topi/reduction.h:47-58) indexes elements of other rows. */
typedef struct kxc_b200_softmax_desc {
    int32_t rank;
    int64_t shape[6];
    int32_t axis; /* negative values count from the end */
} kxc_b200_softmax_desc;
int32_t kxc_b200_softmax(void** packed_args, const kxc_b200_softmax_desc* desc, void* stream);

/* reduce_mean — ReduceMeanCompute (src/relay/op/tensor/reduce.cc:81-99): sequential sum over the reduced axes (nested
 * loops in ascending axis order), then / (float)count. packed_args = { x, out }; out holds the kept dimensions in
 * order (with extent-1 dimensions in place of the reduced ones when keepdims is set). keepdims = 1 is accepted only when
 * the reduced axes are the trailing ones (elsewhere the reference's reduction reads the wrong elements). Bit-exact. */
typedef struct kxc_b200_reduce_desc {
    int32_t rank;
    int64_t shape[6];
    int32_t num_axes;
    int32_t axes[6];
    int32_t keepdims;
} kxc_b200_reduce_desc;
int32_t kxc_b200_reduce_mean(void** packed_args, const kxc_b200_reduce_desc* desc, void* stream);

/* matmul — topi::matmul (include/te/topi/nn.h:82-101) via MatMulCompute (src/relay/op/tensor/math.cc:82-87):
 * out[i,j] = sum over k, in ascending order, of a[i,k] * b[k,j]; rank-2 operands only (MatMulInferType,
 * src/relay/type_infer.cc:280-298). packed_args = { a[M,K], b[K,N], out[M,N] }; precision = KXC_B200_PREC_*. */
int32_t kxc_b200_matmul(void** packed_args, int32_t m, int32_t n, int32_t k, int32_t precision, void* stream);

/* transpose — topi::transpose (include/te/topi/transform.h:20-52) via TransposeCompute
 * (src/relay/op/tensor/transform.cc:206-212): out dimension i is input dimension perm[i]; num_axes = 0 reverses the
 * dimensions; negative axes count from the end (TransposeInferType, src/relay/type_infer.cc:520-548). Elements are moved
 * as bytes, so any dtype of 1, 4 or 8 bytes works. packed_args = { x, out } (not in place). */
typedef struct kxc_b200_transpose_desc {
    int32_t rank;
    int64_t shape[6]; /* of the input */
    int32_t num_axes; /* 0 or rank */
    int32_t perm[6];
    int32_t elem_bytes;
} kxc_b200_transpose_desc;
int32_t kxc_b200_transpose(void** packed_args, const kxc_b200_transpose_desc* desc, void* stream);

/* reshape — ReshapeCompute (src/relay/op/tensor/transform.cc:185-204): the flat element order is unchanged, so this is
 * a copy (a no-op when both pointers are equal). The caller resolves 0 / -1 entries of newshape as ReshapeInferType
 * does (src/relay/type_infer.cc:454-512). packed_args = { x, out }. */
int32_t kxc_b200_reshape(void** packed_args, int64_t numel, int32_t elem_bytes, void* stream);

/* cast — topi::cast (include/te/topi/elemwise.h:113-122) via CastCompute (src/relay/op/tensor/transform.cc:214-224);
 * dtype codes are the reference's CastAttrs codes (DTypeFromCastCode, transform.cc:84-103). Conversion semantics are
 * those of CodeGenLLVM::CastValue (src/codegen/codegen_llvm.cc:219-248). A float outside the integer type's range is
 * undefined in the reference and saturates here; bool (code 4) is refused. packed_args = { x, out }. */
enum {
    KXC_B200_DT_F32 = 0,
    KXC_B200_DT_I32 = 1,
    KXC_B200_DT_I64 = 2,
    KXC_B200_DT_F64 = 3,
    KXC_B200_DT_BOOL = 4,
    KXC_B200_DT_I8 = 5,
    KXC_B200_DT_U8 = 6
};
int32_t kxc_b200_cast(void** packed_args, int64_t numel, int32_t from, int32_t to, void* stream);

/* nn_global_avg_pool2d — topi::global_avg_pool2d (include/te/topi/nn.h:260-287).
 * packed_args = { x[N,C,H,W], out[N,C,1,1] }. The sum runs sequentially over (h,w) per plane, like
 * the reference, so the result is bit-exact. */
int32_t kxc_b200_nn_global_avg_pool2d(void** packed_args, int32_t n, int32_t c, int32_t h, int32_t w, void* stream);

/* nn_flatten — FlattenCompute (src/relay/op/tensor/transform.cc:140-182): a re-indexing copy.
 * packed_args = { x[numel], out[numel] } (no-op when both pointers are equal). */
int32_t kxc_b200_nn_flatten(void** packed_args, int64_t numel, void* stream);

/* nn_dense / nn_gemm — topi::dense (include/te/topi/nn.h:48-80), GemmCompute (src/relay/op/nn/dense.cc:34-61).
 * dense: packed_args = { a[M,K], b[N,K], out[M,N] };  gemm: { a[M,K], b, c[N], out[M,N] } with
 * b = [N,K] when transB=1 else [K,N]; transA must be 0 (the reference throws otherwise). */
typedef struct kxc_b200_gemm_desc {
    int32_t m, n, k;
    float alpha, beta;
    int32_t transA, transB;
    int32_t has_c;     /* 0 = nn_dense, 1 = nn_gemm */
    int32_t precision; /* KXC_B200_PREC_* */
} kxc_b200_gemm_desc;
int32_t kxc_b200_nn_gemm(void** packed_args, const kxc_b200_gemm_desc* desc, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KXC_B200_H_ */

/* kxc_oracle.h — CPU restatement ("port") of the arithmetic the reference compiler
 * (KDZZZZZZ/hdkx-aicompiler) emits for the ResNet-class operator path.
 *
 * TEST INFRASTRUCTURE ONLY: the checker for tests/, the smoke check and bench.py's cpu_baseline leg.
 * The shipped library (libkxc_b200.so) never links, loads or calls anything declared here.
 *
 * Every function follows one reference definition (cited per function in kxc_oracle.c) and keeps its
 * per-element operation order: accumulators start at the reference's identity, reductions run
 * rc -> rh -> rw (or k) sequentially, every multiply and add is a separately rounded fp32 operation
 * (build with -ffp-contract=off). Parity of this port is pinned two ways by tests/test_oracle.py:
 * against the reference's own golden vectors (test/op_numeric_llvm_test.cpp) and, bit for bit, against
 * the C text the unmodified reference compiler generates for the same ops (oracle/_ref/ref_emit).
 *
 * The int8 requantize step and the bf16/tf32 operand roundings have no counterpart in the reference
 * (it has no quantize op and no 16/19-bit float type): for those this header is the definition and
 * parity is "unpinned" beyond the int32 accumulators, which ARE pinned against the reference's
 * nn_conv2d run at int32.
 */
#ifndef KXC_ORACLE_H_
#define KXC_ORACLE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* All tensors dense row-major, NCHW / OIHW, int64 index arithmetic. Return 0 on success. */

int32_t kxc_oracle_conv2d_f32(const float* data, const float* weight, const float* bias /* may be NULL */,
                              float* out, int64_t N, int64_t C, int64_t H, int64_t W, int64_t O,
                              int64_t KH, int64_t KW, int64_t sh, int64_t sw, int64_t ph, int64_t pw,
                              int64_t dh, int64_t dw);

int32_t kxc_oracle_conv2d_i32(const int32_t* data, const int32_t* weight, const int32_t* bias /* may be NULL */,
                              int32_t* out, int64_t N, int64_t C, int64_t H, int64_t W, int64_t O,
                              int64_t KH, int64_t KW, int64_t sh, int64_t sw, int64_t ph, int64_t pw,
                              int64_t dh, int64_t dw);

/* int8 activations/weights, int32 accumulate + int32 bias, fixed-point requantize to int8.
 * acc_out (optional, may be NULL) receives the int32 accumulators after the bias add. */
int32_t kxc_oracle_conv2d_s8_requant(const int8_t* data, const int8_t* weight, const int32_t* bias,
                                     const int32_t* multiplier, const int32_t* shift, int32_t relu,
                                     int8_t* out, int32_t* acc_out, int64_t N, int64_t C, int64_t H,
                                     int64_t W, int64_t O, int64_t KH, int64_t KW, int64_t sh, int64_t sw,
                                     int64_t ph, int64_t pw, int64_t dh, int64_t dw);

/* One accumulator through the requantize definition (exposed for unit tests). */
int8_t kxc_oracle_requant_one(int32_t acc, int32_t multiplier, int32_t shift, int32_t relu);

int32_t kxc_oracle_relu_f32(const float* x, float* out, int64_t n);

/* NumPy-style right-aligned broadcast add; shapes padded on the left with 1s to `rank` (<= 6). */
int32_t kxc_oracle_add_f32(const float* a, const int64_t* a_shape, const float* b, const int64_t* b_shape,
                           float* out, const int64_t* out_shape, int32_t rank);

int32_t kxc_oracle_max_pool2d_f32(const float* x, float* out, int64_t N, int64_t C, int64_t H, int64_t W,
                                  int64_t KH, int64_t KW, int64_t sh, int64_t sw, int64_t pt, int64_t pl,
                                  int64_t pb, int64_t pr, int32_t ceil_mode);

int32_t kxc_oracle_avg_pool2d_f32(const float* x, float* out, int64_t N, int64_t C, int64_t H, int64_t W,
                                  int64_t KH, int64_t KW, int64_t sh, int64_t sw, int64_t pt, int64_t pl,
                                  int64_t pb, int64_t pr, int32_t ceil_mode);

int32_t kxc_oracle_global_avg_pool2d_f32(const float* x, float* out, int64_t N, int64_t C, int64_t H, int64_t W);
int32_t kxc_oracle_softmax_f32(const float* x, float* out, int64_t outer, int64_t len, int64_t inner);
int32_t kxc_oracle_reduce_mean_f32(const float* x, float* out, int32_t rank, const int64_t* shape, const int32_t* reduce);

/* out[i,j] = sum_k a[i,k]*b[j,k]  (b is [Nn,K]) */
int32_t kxc_oracle_dense_f32(const float* a, const float* b, float* out, int64_t M, int64_t Nn, int64_t K);

int32_t kxc_oracle_matmul_f32(const float* a, const float* b, float* out, int64_t M, int64_t Nn, int64_t K);
int32_t kxc_oracle_transpose(const void* x, void* out, int32_t rank, const int64_t* shape, const int32_t* perm, int32_t elem);
int32_t kxc_oracle_cast(const void* x, void* out, int64_t n, int32_t from, int32_t to);

/* nn_gemm: transA must be 0; transB=1 -> b is [Nn,K], transB=0 -> b is [K,Nn]; c broadcast [Nn]. */
int32_t kxc_oracle_gemm_f32(const float* a, const float* b, const float* c, float* out, int64_t M, int64_t Nn,
                            int64_t K, float alpha, float beta, int32_t transA, int32_t transB);

/* Pooling output extent, floor or ceil mode (include/te/topi/nn.h:201-204). */
int64_t kxc_oracle_pool_out_dim(int64_t in, int64_t k, int64_t s, int64_t p0, int64_t p1, int32_t ceil_mode);
/* Convolution output extent (include/te/topi/nn.h:118-124). */
int64_t kxc_oracle_conv_out_dim(int64_t in, int64_t k, int64_t s, int64_t p, int64_t d);

/* Operand roundings used by the reduced-precision modes (no reference counterpart). */
void kxc_oracle_round_bf16(const float* x, float* out, int64_t n); /* fp32 -> bf16 RNE -> fp32 */
void kxc_oracle_round_tf32(const float* x, float* out, int64_t n); /* fp32 -> tf32 RNE (10-bit mantissa) -> fp32 */

#ifdef __cplusplus
}
#endif
#endif /* KXC_ORACLE_H_ */

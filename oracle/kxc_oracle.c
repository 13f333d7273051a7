/* kxc_oracle.c — CPU restatement of the reference operator arithmetic. TEST INFRASTRUCTURE ONLY
 * (see kxc_oracle.h). Build: gcc -O2 -ffp-contract=off -fno-fast-math (no FMA contraction: the
 * reference's LLVM backend emits separate fmul/fadd without contract flags,
 * src/codegen/codegen_llvm.cc:295-305).
 *
 * Reduction identities and loop nesting follow src/relay/backend/lower.cc:389-449 (init; then
 * `out = out (+) src` over the reduce axes in declaration order) and :73-95 (sum -> 0, max -> -inf).
 * Loops over output elements are free to be reordered because every output element is an independent
 * sequential reduction; only the order INSIDE one element's reduction matters for the bits.
 */
#include "kxc_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

int64_t kxc_oracle_conv_out_dim(int64_t in, int64_t k, int64_t s, int64_t p, int64_t d) {
    /* include/te/topi/nn.h:118-124: OH = (H + 2*pad - ((KH-1)*dil + 1)) / stride + 1 */
    return (in + 2 * p - ((k - 1) * d + 1)) / s + 1;
}

int64_t kxc_oracle_pool_out_dim(int64_t in, int64_t k, int64_t s, int64_t p0, int64_t p1, int32_t ceil_mode) {
    /* include/te/topi/nn.h:201-204 */
    int64_t num = in + p0 + p1 - k;
    return ceil_mode ? ((num + s - 1) / s + 1) : (num / s + 1);
}

/* ---- nn_conv2d: include/te/topi/nn.h:107-158 (conv2d_nchw) + src/relay/op/nn/convolution.cc:66-74
 * (separate bias-add pass). acc = 0; for rc, rh, rw: acc = acc + (inb ? x : 0) * w; out = acc + bias.
 * The innermost loop here runs over an output ROW (ow) with one accumulator per element, so each
 * element still sees rc -> rh -> rw order; a padded tap contributes acc + 0*w like the reference. */
#define KXC_CONV_BODY(T, ZERO)                                                                          \
    const int64_t OH = kxc_oracle_conv_out_dim(H, KH, sh, ph, dh);                                      \
    const int64_t OW = kxc_oracle_conv_out_dim(W, KW, sw, pw, dw);                                      \
    if (OH <= 0 || OW <= 0) return 1;                                                                   \
    T* acc = (T*)malloc(sizeof(T) * (size_t)OW);                                                        \
    if (!acc) return 2;                                                                                 \
    for (int64_t n = 0; n < N; ++n)                                                                     \
        for (int64_t o = 0; o < O; ++o)                                                                 \
            for (int64_t oh = 0; oh < OH; ++oh) {                                                       \
                for (int64_t ow = 0; ow < OW; ++ow) acc[ow] = ZERO;                                     \
                for (int64_t rc = 0; rc < C; ++rc)                                                      \
                    for (int64_t rh = 0; rh < KH; ++rh) {                                               \
                        const int64_t ih = oh * sh + rh * dh - ph;                                      \
                        const int inb_h = (ih >= 0) && (ih < H);                                        \
                        const T* xrow = data + ((n * C + rc) * H + (inb_h ? ih : 0)) * W;               \
                        for (int64_t rw = 0; rw < KW; ++rw) {                                           \
                            const T wv = weight[((o * C + rc) * KH + rh) * KW + rw];                    \
                            for (int64_t ow = 0; ow < OW; ++ow) {                                       \
                                const int64_t iw = ow * sw + rw * dw - pw;                              \
                                const T xv = (inb_h && iw >= 0 && iw < W) ? xrow[iw] : ZERO;            \
                                acc[ow] = acc[ow] + xv * wv;                                            \
                            }                                                                           \
                        }                                                                               \
                    }                                                                                   \
                T* orow = out + ((n * O + o) * OH + oh) * OW;                                           \
                if (bias)                                                                               \
                    for (int64_t ow = 0; ow < OW; ++ow) orow[ow] = acc[ow] + bias[o];                   \
                else                                                                                    \
                    for (int64_t ow = 0; ow < OW; ++ow) orow[ow] = acc[ow];                             \
            }                                                                                           \
    free(acc);                                                                                          \
    return 0;

int32_t kxc_oracle_conv2d_f32(const float* data, const float* weight, const float* bias, float* out, int64_t N,
                              int64_t C, int64_t H, int64_t W, int64_t O, int64_t KH, int64_t KW, int64_t sh,
                              int64_t sw, int64_t ph, int64_t pw, int64_t dh, int64_t dw) {
    KXC_CONV_BODY(float, 0.0f)
}

int32_t kxc_oracle_conv2d_i32(const int32_t* data, const int32_t* weight, const int32_t* bias, int32_t* out,
                              int64_t N, int64_t C, int64_t H, int64_t W, int64_t O, int64_t KH, int64_t KW,
                              int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t dh, int64_t dw) {
    KXC_CONV_BODY(int32_t, 0)
}

/* ---- int8 requantize: no reference counterpart; this is the definition the CUDA epilogue matches.
 *   t = (int64)acc * (int64)M;  S = 31 + shift;  q = (t + (1 << (S-1))) >> S   (arithmetic shift:
 *   round half toward +inf);  relu ? q = max(q,0) : q = max(q,-128);  y = (int8)min(q,127). */
int8_t kxc_oracle_requant_one(int32_t acc, int32_t multiplier, int32_t shift, int32_t relu) {
    const int64_t t = (int64_t)acc * (int64_t)multiplier;
    const int S = 31 + shift;
    int64_t q = (t + ((int64_t)1 << (S - 1))) >> S;
    const int64_t lo = relu ? 0 : -128;
    if (q < lo) q = lo;
    if (q > 127) q = 127;
    return (int8_t)q;
}

int32_t kxc_oracle_conv2d_s8_requant(const int8_t* data, const int8_t* weight, const int32_t* bias,
                                     const int32_t* multiplier, const int32_t* shift, int32_t relu, int8_t* out,
                                     int32_t* acc_out, int64_t N, int64_t C, int64_t H, int64_t W, int64_t O,
                                     int64_t KH, int64_t KW, int64_t sh, int64_t sw, int64_t ph, int64_t pw,
                                     int64_t dh, int64_t dw) {
    /* accumulators: exactly nn_conv2d (+bias) on the int8 values widened to int32 */
    const int64_t OH = kxc_oracle_conv_out_dim(H, KH, sh, ph, dh);
    const int64_t OW = kxc_oracle_conv_out_dim(W, KW, sw, pw, dw);
    if (OH <= 0 || OW <= 0) return 1;
    int32_t* acc = (int32_t*)malloc(sizeof(int32_t) * (size_t)OW);
    if (!acc) return 2;
    for (int64_t n = 0; n < N; ++n)
        for (int64_t o = 0; o < O; ++o)
            for (int64_t oh = 0; oh < OH; ++oh) {
                for (int64_t ow = 0; ow < OW; ++ow) acc[ow] = 0;
                for (int64_t rc = 0; rc < C; ++rc)
                    for (int64_t rh = 0; rh < KH; ++rh) {
                        const int64_t ih = oh * sh + rh * dh - ph;
                        if (ih < 0 || ih >= H) continue; /* integer: adding 0 is exact, skip */
                        const int8_t* xrow = data + ((n * C + rc) * H + ih) * W;
                        for (int64_t rw = 0; rw < KW; ++rw) {
                            const int32_t wv = weight[((o * C + rc) * KH + rh) * KW + rw];
                            for (int64_t ow = 0; ow < OW; ++ow) {
                                const int64_t iw = ow * sw + rw * dw - pw;
                                if (iw >= 0 && iw < W) acc[ow] += (int32_t)xrow[iw] * wv;
                            }
                        }
                    }
                const int64_t base = ((n * O + o) * OH + oh) * OW;
                for (int64_t ow = 0; ow < OW; ++ow) {
                    const int32_t a = acc[ow] + (bias ? bias[o] : 0);
                    if (acc_out) acc_out[base + ow] = a;
                    out[base + ow] = kxc_oracle_requant_one(a, multiplier[o], shift[o], relu);
                }
            }
    free(acc);
    return 0;
}

/* ---- nn_relu: include/te/topi/nn.h:19-30; Max(x,0) lowers to `x > 0 ? x : 0`
 * (src/codegen/codegen_llvm.cc:326-333): NaN -> 0, -0 -> +0. */
int32_t kxc_oracle_relu_f32(const float* x, float* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = (x[i] > 0.0f) ? x[i] : 0.0f;
    return 0;
}

/* ---- add: include/te/topi/broadcast.h:18-41,90-109. Input dim == 1 -> index 0, else output index. */
int32_t kxc_oracle_add_f32(const float* a, const int64_t* a_shape, const float* b, const int64_t* b_shape,
                           float* out, const int64_t* out_shape, int32_t rank) {
    if (rank < 1 || rank > 6) return 1;
    int64_t total = 1;
    for (int i = 0; i < rank; ++i) total *= out_shape[i];
    int64_t idx[6] = {0, 0, 0, 0, 0, 0};
    for (int64_t lin = 0; lin < total; ++lin) {
        int64_t ai = 0, bi = 0;
        for (int i = 0; i < rank; ++i) {
            ai = ai * a_shape[i] + (a_shape[i] == 1 ? 0 : idx[i]);
            bi = bi * b_shape[i] + (b_shape[i] == 1 ? 0 : idx[i]);
        }
        out[lin] = a[ai] + b[bi];
        for (int i = rank - 1; i >= 0; --i) {
            if (++idx[i] < out_shape[i]) break;
            idx[i] = 0;
        }
    }
    return 0;
}

/* ---- nn_max_pool2d: include/te/topi/nn.h:161-229. m = -inf; v = inb ? x : -1e30f; m = m > v ? m : v. */
int32_t kxc_oracle_max_pool2d_f32(const float* x, float* out, int64_t N, int64_t C, int64_t H, int64_t W,
                                  int64_t KH, int64_t KW, int64_t sh, int64_t sw, int64_t pt, int64_t pl,
                                  int64_t pb, int64_t pr, int32_t ceil_mode) {
    const int64_t OH = kxc_oracle_pool_out_dim(H, KH, sh, pt, pb, ceil_mode);
    const int64_t OW = kxc_oracle_pool_out_dim(W, KW, sw, pl, pr, ceil_mode);
    if (OH <= 0 || OW <= 0) return 1;
    const float pad_value = (float)-1e30; /* make_const(float32, -1e30), nn.h:224 */
    for (int64_t nc = 0; nc < N * C; ++nc)
        for (int64_t oh = 0; oh < OH; ++oh)
            for (int64_t ow = 0; ow < OW; ++ow) {
                float m = -INFINITY;
                for (int64_t rh = 0; rh < KH; ++rh)
                    for (int64_t rw = 0; rw < KW; ++rw) {
                        const int64_t ih = oh * sh + rh - pt, iw = ow * sw + rw - pl;
                        const float v =
                            (ih >= 0 && ih < H && iw >= 0 && iw < W) ? x[(nc * H + ih) * W + iw] : pad_value;
                        m = (m > v) ? m : v;
                    }
                out[(nc * OH + oh) * OW + ow] = m;
            }
    return 0;
}

/* ---- nn_avg_pool2d: include/te/topi/nn.h:231-257. s = 0; s += inb ? x : 0; out = s / (float)(KH*KW). */
int32_t kxc_oracle_avg_pool2d_f32(const float* x, float* out, int64_t N, int64_t C, int64_t H, int64_t W,
                                  int64_t KH, int64_t KW, int64_t sh, int64_t sw, int64_t pt, int64_t pl,
                                  int64_t pb, int64_t pr, int32_t ceil_mode) {
    const int64_t OH = kxc_oracle_pool_out_dim(H, KH, sh, pt, pb, ceil_mode);
    const int64_t OW = kxc_oracle_pool_out_dim(W, KW, sw, pl, pr, ceil_mode);
    if (OH <= 0 || OW <= 0) return 1;
    const float div = (float)(KH * KW);
    for (int64_t nc = 0; nc < N * C; ++nc)
        for (int64_t oh = 0; oh < OH; ++oh)
            for (int64_t ow = 0; ow < OW; ++ow) {
                float s = 0.0f;
                for (int64_t rh = 0; rh < KH; ++rh)
                    for (int64_t rw = 0; rw < KW; ++rw) {
                        const int64_t ih = oh * sh + rh - pt, iw = ow * sw + rw - pl;
                        const float v = (ih >= 0 && ih < H && iw >= 0 && iw < W) ? x[(nc * H + ih) * W + iw] : 0.0f;
                        s = s + v;
                    }
                out[(nc * OH + oh) * OW + ow] = s / div;
            }
    return 0;
}

/* ---- nn_global_avg_pool2d: include/te/topi/nn.h:260-287. s = 0; s += x over rh, rw; out = s / (H*W)
 * (true division; the integer extent converts to float). */
int32_t kxc_oracle_global_avg_pool2d_f32(const float* x, float* out, int64_t N, int64_t C, int64_t H, int64_t W) {
    const float div = (float)(H * W);
    for (int64_t nc = 0; nc < N * C; ++nc) {
        float s = 0.0f;
        for (int64_t i = 0; i < H * W; ++i) s = s + x[nc * H * W + i];
        out[nc] = s / div;
    }
    return 0;
}

/* ---- softmax: src/relay/op/nn/softmax.cc:44-70. e = exp(x) elementwise (expf of the C library), s = 0; s = s + e over
 * the axis in index order; out = e / s. No subtraction of the maximum. x is viewed as [outer, len, inner]. */
int32_t kxc_oracle_softmax_f32(const float* x, float* out, int64_t outer, int64_t len, int64_t inner) {
    for (int64_t o = 0; o < outer; ++o)
        for (int64_t i = 0; i < inner; ++i) {
            const float* xp = x + o * len * inner + i;
            float* op = out + o * len * inner + i;
            float s = 0.0f;
            for (int64_t k = 0; k < len; ++k) s = s + expf(xp[k * inner]);
            for (int64_t k = 0; k < len; ++k) op[k * inner] = expf(xp[k * inner]) / s;
        }
    return 0;
}

/* ---- reduce_mean: src/relay/op/tensor/reduce.cc:81-99 over topi::sum (include/te/topi/reduction.h:23-70). s = 0;
 * s = s + x with the reduced axes as nested loops in ascending axis order; out = s / (float)count. `reduce[d]` marks
 * the reduced dimensions of the rank-`rank` row-major input; the output is the kept dimensions in order. */
int32_t kxc_oracle_reduce_mean_f32(const float* x, float* out, int32_t rank, const int64_t* shape, const int32_t* reduce) {
    int64_t stride[8], kept[8], red[8];
    int nk = 0, nr = 0;
    int64_t st = 1, count = 1, nout = 1;
    if (rank < 0 || rank > 8) return 1;
    for (int d = rank - 1; d >= 0; --d) { stride[d] = st; st *= shape[d]; }
    for (int d = 0; d < rank; ++d) {
        if (reduce[d]) { red[nr++] = d; count *= shape[d]; } else { kept[nk++] = d; nout *= shape[d]; }
    }
    for (int64_t o = 0; o < nout; ++o) {
        int64_t rem = o, base = 0;
        for (int j = nk - 1; j >= 0; --j) { base += (rem % shape[kept[j]]) * stride[kept[j]]; rem /= shape[kept[j]]; }
        float s = 0.0f;
        for (int64_t r = 0; r < count; ++r) {
            int64_t rr = r, off = base;
            for (int j = nr - 1; j >= 0; --j) { off += (rr % shape[red[j]]) * stride[red[j]]; rr /= shape[red[j]]; }
            s = s + x[off];
        }
        out[o] = s / (float)count;
    }
    return 0;
}

/* ---- nn_dense: include/te/topi/nn.h:48-80. acc = 0; acc += a[i,k] * b[j,k]. */
int32_t kxc_oracle_dense_f32(const float* a, const float* b, float* out, int64_t M, int64_t Nn, int64_t K) {
    for (int64_t i = 0; i < M; ++i)
        for (int64_t j = 0; j < Nn; ++j) {
            float acc = 0.0f;
            for (int64_t k = 0; k < K; ++k) acc = acc + a[i * K + k] * b[j * K + k];
            out[i * Nn + j] = acc;
        }
    return 0;
}

/* ---- nn_gemm: src/relay/op/nn/dense.cc:34-61. dense (transB=1) or matmul (transB=0,
 * include/te/topi/nn.h:84-101); then *alpha if alpha != 1; bias*beta if beta != 1; then + bias[j]. */
int32_t kxc_oracle_gemm_f32(const float* a, const float* b, const float* c, float* out, int64_t M, int64_t Nn,
                            int64_t K, float alpha, float beta, int32_t transA, int32_t transB) {
    if (transA != 0) return 1; /* the reference throws for transA=1 */
    for (int64_t i = 0; i < M; ++i)
        for (int64_t j = 0; j < Nn; ++j) {
            float acc = 0.0f;
            if (transB == 1)
                for (int64_t k = 0; k < K; ++k) acc = acc + a[i * K + k] * b[j * K + k];
            else
                for (int64_t k = 0; k < K; ++k) acc = acc + a[i * K + k] * b[k * Nn + j];
            if ((double)alpha != 1.0) acc = acc * alpha;
            float bias = c[j];
            if ((double)beta != 1.0) bias = bias * beta;
            out[i * Nn + j] = acc + bias;
        }
    return 0;
}

/* ---- matmul: include/te/topi/nn.h:82-101. acc = 0; acc = acc + a[i,k] * b[k,j], k ascending. ---- */
int32_t kxc_oracle_matmul_f32(const float* a, const float* b, float* out, int64_t M, int64_t Nn, int64_t K) {
    for (int64_t i = 0; i < M; ++i)
        for (int64_t j = 0; j < Nn; ++j) {
            float acc = 0.0f;
            for (int64_t k = 0; k < K; ++k) acc = acc + a[i * K + k] * b[k * Nn + j];
            out[i * Nn + j] = acc;
        }
    return 0;
}

/* ---- transpose: include/te/topi/transform.h:20-52. Output dimension i has the extent of input dimension perm[i]; the
 * input index along perm[i] is the output index along i. Elements are `elem` bytes wide. ---- */
int32_t kxc_oracle_transpose(const void* x, void* out, int32_t rank, const int64_t* shape, const int32_t* perm, int32_t elem) {
    int64_t istride[8], oshape[8], idx[8], total = 1;
    if (rank < 1 || rank > 8) return 1;
    int64_t st = 1;
    for (int i = rank - 1; i >= 0; --i) {
        istride[i] = st;
        st *= shape[i];
    }
    for (int i = 0; i < rank; ++i) {
        oshape[i] = shape[perm[i]];
        total *= oshape[i];
        idx[i] = 0;
    }
    const char* src = (const char*)x;
    char* dst = (char*)out;
    for (int64_t o = 0; o < total; ++o) {
        int64_t off = 0;
        for (int i = 0; i < rank; ++i) off += idx[i] * istride[perm[i]];
        memcpy(dst + o * elem, src + off * elem, (size_t)elem);
        for (int i = rank - 1; i >= 0; --i) {
            if (++idx[i] < oshape[i]) break;
            idx[i] = 0;
        }
    }
    return 0;
}

/* ---- cast: include/te/topi/elemwise.h:113-122, scalar rule CodeGenLLVM::CastValue (src/codegen/codegen_llvm.cc:219-248).
 * dtype codes as in DTypeFromCastCode (src/relay/op/tensor/transform.cc:84-103): 0 f32, 1 i32, 2 i64, 3 f64, 5 i8, 6 u8.
 * Every pair below is the C conversion, which is what sext/zext/trunc, sitofp/uitofp, fptosi/fptoui and fpext/fptrunc
 * compute for values the target can hold (a float outside an integer target's range is undefined there and here). ---- */
#define KXC_CAST_LOOP(S, D)                                             \
    {                                                                   \
        const S* s_ = (const S*)x;                                      \
        D* d_ = (D*)out;                                                \
        for (int64_t i = 0; i < n; ++i) d_[i] = (D)s_[i];               \
        return 0;                                                       \
    }
#define KXC_CAST_TO(S)                                   \
    switch (to) {                                        \
        case 0: KXC_CAST_LOOP(S, float)                  \
        case 1: KXC_CAST_LOOP(S, int32_t)                \
        case 2: KXC_CAST_LOOP(S, int64_t)                \
        case 3: KXC_CAST_LOOP(S, double)                 \
        case 5: KXC_CAST_LOOP(S, int8_t)                 \
        case 6: KXC_CAST_LOOP(S, uint8_t)                \
        default: return 1;                               \
    }
int32_t kxc_oracle_cast(const void* x, void* out, int64_t n, int32_t from, int32_t to) {
    switch (from) {
        case 0: KXC_CAST_TO(float)
        case 1: KXC_CAST_TO(int32_t)
        case 2: KXC_CAST_TO(int64_t)
        case 3: KXC_CAST_TO(double)
        case 5: KXC_CAST_TO(int8_t)
        case 6: KXC_CAST_TO(uint8_t)
        default: return 1;
    }
}

/* ---- operand roundings for the reduced-precision modes (no reference counterpart) ---- */
void kxc_oracle_round_bf16(const float* x, float* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        uint32_t u;
        memcpy(&u, &x[i], 4);
        if ((u & 0x7fffffffu) > 0x7f800000u) {
            u = (u | 0x00400000u) & 0xffff0000u; /* quiet NaN */
        } else {
            u = (u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u; /* round to nearest even */
        }
        memcpy(&out[i], &u, 4);
    }
}

void kxc_oracle_round_tf32(const float* x, float* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        uint32_t u;
        memcpy(&u, &x[i], 4);
        if ((u & 0x7f800000u) != 0x7f800000u) {
            u = (u + 0xfffu + ((u >> 13) & 1u)) & 0xffffe000u; /* keep 10 mantissa bits, RNE */
        }
        memcpy(&out[i], &u, 4);
    }
}

// Types shared by the convolution / GEMM translation units.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "kxc_b200.h"

namespace kxc_b200 {

struct ConvDims {
    int N, C, H, W;
    int O, KH, KW;
    int SH, SW, PH, PW, DH, DW;
    int OH, OW;
};

// Fixed-point requantize of one int32 accumulator to int8 (the library's definition; the reference
// has no quantized op):  q = (acc*M + 2^(S-1)) >> S  with S = 31 + shift, 64-bit, arithmetic shift
// (round half toward +inf);  relu ? max(q,0) : max(q,-128);  min(q,127).
__host__ __device__ __forceinline__ int8_t requantize_s8(int32_t acc, int32_t multiplier, int32_t shift, int relu) {
    const long long t = (long long)acc * (long long)multiplier;
    const int S = 31 + shift;
    long long q = (t + (1LL << (S - 1))) >> S;
    const long long lo = relu ? 0 : -128;
    q = q < lo ? lo : q;
    q = q > 127 ? 127 : q;
    return (int8_t)q;
}

// conv_simt.cu
int32_t conv2d_fp32_exact(const float* data, const float* weight, const float* bias, const float* residual, float* out,
                          const ConvDims& d, int relu, cudaStream_t s);
int32_t conv2d_s8_exact(const int8_t* data, const int8_t* weight, const int32_t* bias, const int32_t* multiplier,
                        const int32_t* shift, int8_t* out, const ConvDims& d, int relu, cudaStream_t s);
int32_t gemm_fp32_exact(const float* a, const float* b, const float* c, float* out, const kxc_b200_gemm_desc& g,
                        cudaStream_t s);


// conv_tc_api.cu: reference-layout tensors -> tensor-core implicit GEMM (falls back to the CUDA-core
// kernels for shapes the tensor-core path does not take)
int32_t conv2d_tensor_core(const float* data, const float* weight, const float* bias, const float* residual, float* out,
                           const ConvDims& d, int relu, int precision, cudaStream_t s);
int32_t conv2d_s8_dispatch(const int8_t* data, const int8_t* weight, const int32_t* bias, const int32_t* multiplier,
                           const int32_t* shift, int8_t* out, const ConvDims& d, int relu, int force_simt, int nhwc, cudaStream_t s);
int32_t gemm_tensor_core(const float* a, const float* b, const float* c, float* out, const kxc_b200_gemm_desc& g,
                         cudaStream_t s);

}  // namespace kxc_b200

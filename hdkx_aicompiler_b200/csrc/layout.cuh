// Layout / precision conversions at the edges of the tensor-core path.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "conv_tc.cuh"

namespace kxc_b200 {

// NCHW (fp32 or int8) -> NHWC with `cpad` channels (zero filled), converted to the tensor-core
// operand type: bf16 (round to nearest even), tf32 kept in fp32 storage (low 13 mantissa bits
// rounded away, nearest even), or int8 (copied).
int32_t nchw_to_nhwc(const void* in, void* out, TcDType dtype, int N, int C, int HW, int cpad, cudaStream_t s, bool tf32_lo = false);

// int8 NCHW -> NHWC of only the pixels a 1x1 convolution of stride `stride` without padding reads:
// out[n][oh][ow][c] = in[n][c][oh*stride][ow*stride], channels zero-filled up to cpad (a multiple of 4).
int32_t nchw_to_nhwc_s8_subsample(const int8_t* in, int8_t* out, int N, int C, int H, int W, int OH, int OW, int stride, int cpad,
                                  cudaStream_t s);

// int8 NHWC [N][HW][C] -> NCHW [N][C][HW] (the reference layout of a requantized result).
int32_t nhwc_to_nchw_s8(const int8_t* in, int8_t* out, int N, int C, int HW, cudaStream_t s);

// OIHW (fp32 or int8) -> [O][KH][KW][cpad] in the operand type.
int32_t pack_weights_ohwi(const void* w, void* out, TcDType dtype, int O, int C, int KH, int KW, int cpad, cudaStream_t s, bool tf32_lo = false);

// Row-major [rows, cols] fp32 -> [rows, cpad] operand type (dense operands).
int32_t convert_rows(const float* in, void* out, TcDType dtype, int64_t rows, int cols, int cpad, cudaStream_t s, bool tf32_lo = false);

}  // namespace kxc_b200

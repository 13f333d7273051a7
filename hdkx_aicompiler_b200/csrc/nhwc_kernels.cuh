// Kernels on the executor's internal NHWC activation format (bf16 or fp32 storage).
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "conv_tc.cuh"

namespace kxc_b200 {

int32_t maxpool_nhwc(const void* x, void* out, TcDType dt, int N, int H, int W, int C, int OH, int OW, int KH, int KW, int SH,
                     int SW, int PT, int PL, cudaStream_t s);
int32_t gap_nhwc(const void* x, void* out, TcDType dt, int N, int HW, int C, cudaStream_t s);
// out = relu?(a + b); b == nullptr gives a plain relu
int32_t eltwise_nhwc(const void* a, const void* b, void* out, TcDType dt, int64_t numel, int relu, cudaStream_t s);
int32_t nhwc_to_nchw_f32(const void* in, float* out, TcDType dt, int N, int C, int HW, cudaStream_t s);
// Stem (few-channel, stride-2) input packing and its weight packing; see plan.cu.
int32_t stem_pack(const float* x, void* out, TcDType dt, int N, int C, int H, int W, int Hp, int Wp, int pad_h, int pad_w,
                  cudaStream_t s);
int32_t stem_pack_weights(const float* w, void* out, TcDType dt, int O, int C, int KH, int KW, cudaStream_t s);

}  // namespace kxc_b200

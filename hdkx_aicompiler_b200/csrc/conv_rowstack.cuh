// 3x3 stride-1 convolution for 64 -> 64 channel bf16 NHWC layers with the three filter rows stacked along the MMA's
// N dimension (12 instructions of N = 192 per tile instead of 36 of N = 64). See conv_rowstack.cu.
#pragma once

#include "conv_tc.cuh"

namespace kxc_b200 {

bool rowstack3x3_applicable(TcDType dtype, int C, int O, int KH, int KW, int stride, int pad_h, int pad_w, int dil_h, int dil_w,
                            int H, int W);
// Fills geometry and tensor maps of `p` (epilogue pointers are the caller's, as for tc_setup_conv).
int32_t rowstack3x3_setup(TcParams* p, const void* act_nhwc, const void* w_packed, int N, int H, int W);
// Builds the tensor maps of the residual (loads) and output (stores) tensors from p->residual / p->out; call once
// those pointers are final, before the first launch.
int32_t rowstack3x3_bind(TcParams* p);
int32_t rowstack3x3_launch(const TcParams& p, cudaStream_t stream);

// 128 -> 128 channel form on CTA pairs with resident weights (conv_rowstack128.cu); same calling sequence.
bool rowstack128_applicable(TcDType dtype, int C, int O, int KH, int KW, int stride, int pad_h, int pad_w, int dil_h, int dil_w);
int32_t rowstack128_setup(TcParams* p, const void* act_nhwc, const void* w_packed, int N, int H, int W);
int32_t rowstack128_bind(TcParams* p);
int32_t rowstack128_launch(const TcParams& p, cudaStream_t stream);

// int8 form (kind::i8, requantized int8 NHWC result written by the epilogue threads; no residual). The caller fills
// bias_i32 / multiplier / shift / out / relu and calls tc_finish_params before the launch.
bool rowstack3x3_s8_applicable(int C, int O, int KH, int KW, int stride, int pad_h, int pad_w, int dil_h, int dil_w);
int32_t rowstack3x3_s8_setup(TcParams* p, const void* act_nhwc, const void* w_packed, int N, int H, int W);
int32_t rowstack3x3_s8_launch(const TcParams& p, cudaStream_t stream);

}  // namespace kxc_b200

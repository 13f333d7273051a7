// Direct 3x3 stride-1 convolution for 64 -> 64 channel bf16 NHWC layers (resident weights, one halo
// load per tile, shifted shared-memory views as A operands). See conv_direct.cu.
#pragma once

#include "conv_tc.cuh"

namespace kxc_b200 {

bool direct3x3_applicable(TcDType dtype, int C, int O, int KH, int KW, int stride, int pad_h, int pad_w, int dil_h, int dil_w,
                          int OW);
// Fills geometry and tensor maps of `p` (epilogue pointers are the caller's, as for tc_setup_conv).
int32_t direct3x3_setup(TcParams* p, const void* act_nhwc, const void* w_packed, int N, int H, int W);
int32_t direct3x3_launch(const TcParams& p, cudaStream_t stream);

}  // namespace kxc_b200

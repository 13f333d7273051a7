// Direct stride-2 stem convolution on the packed [N][Hp][Wp][4] bf16 layout (see conv_stem.cu).
#pragma once

#include "conv_tc.cuh"

namespace kxc_b200 {

bool stem_direct_applicable(TcDType dtype, int C, int O, int KH, int KW, int OW, int Wp);
size_t stem_direct_weight_bytes(int KH);
// OIHW fp32 -> [KH][4][64][8] bf16 core-matrix order
int32_t stem_direct_pack_weights(const float* w, void* out, int O, int C, int KH, int KW, cudaStream_t s);
int32_t stem_direct_setup(TcParams* p, const void* packed_in, const void* packed_w, int N, int OH, int OW, int KH, int Hp, int Wp);
int32_t stem_direct_launch(const TcParams& p, cudaStream_t stream);
// int8 form of the same kernel (tcgen05 kind::i8, int32 accumulate, fixed-point requantize): packed pixels hold 8 int8
// channels. stem_direct_s8_pack writes the packed input [N][Hp][Wp][8] and the core-matrix weights; the launch takes the
// parameters stem_direct_setup fills plus bias_i32 / multiplier / shift / out / relu.
bool stem_direct_s8_applicable(int C, int O, int KH, int KW, int stride, int dil, int W, int OW, int Wp);
int32_t stem_direct_s8_pack(const int8_t* x, const int8_t* w, void* packed_x, void* packed_w, int N, int C, int H, int W, int O, int KH,
                            int KW, int Hp, int Wp, int pad_h, int pad_w, bool nhwc, cudaStream_t s);
int32_t stem_direct_s8_launch(const TcParams& p, bool nhwc_out, cudaStream_t stream);
// Fused variant: conv + bias + ReLU + max_pool2d(3x3, s2, p1); `p.out` is the POOLED bf16 NHWC tensor
// [N, OH/2, OW/2, 64], p.OH / p.OW stay the convolution's output extent. Same setup as stem_direct_setup.
bool stem_pool_applicable(int OH, int OW, int pool_k, int pool_s, int pool_pad);
int32_t stem_pool_launch(const TcParams& p, cudaStream_t stream);

// conv_stem_fused.cu: the same convolution + bias + ReLU + max_pool2d(3x3, s2, p1), reading the NCHW fp32 graph
// input directly (the packed layout exists only in shared memory) and issuing row-stacked MMAs. `p.aux_in` is the
// fp32 input (bound at run time), `p.out` the pooled bf16 NHWC tensor. Bit-identical to stem_pool_launch.
bool stem_pool_nchw_applicable(TcDType dtype, int C, int O, int KH, int KW, int W, int OH, int OW, int Wp);
size_t stem_stacked_weight_bytes();
// OIHW fp32 -> filter rows stacked by parity in core-matrix order
int32_t stem_stacked_pack_weights(const float* w, void* out, int O, int C, int KW, cudaStream_t s);
int32_t stem_pool_nchw_setup(TcParams* p, const void* packed_w, int N, int C, int H, int W, int OH, int OW, int pad_h, int pad_w,
                             int Hp, int Wp);
int32_t stem_pool_nchw_launch(const TcParams& p, cudaStream_t stream);

}  // namespace kxc_b200

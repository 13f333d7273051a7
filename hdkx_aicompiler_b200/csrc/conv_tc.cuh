// Implicit-GEMM convolution / dense kernel on the 5th-generation tensor cores (tcgen05 + TMEM),
// operands fed by TMA tiled loads. Interface between the kernel TU and its callers.
//
// GEMM view:  D[M = N*OH*OW, Cout] = A[M, K = KH*KW*Cpad] x B[Cout, K]^T
//   activations NHWC (channel-innermost, Cpad channels), weights [Cout][KH][KW][Cpad], both K-major.
//   One CTA tile = 128 output pixels (a BNI x BH x BW box of images x rows x cols) x BN channels.
//   One pipeline stage = one filter tap x one block of `kb_elems` channels: the A tile of that stage
//   is a single 4-D TMA box of the activation tensor shifted by the tap offset; out-of-bounds
//   pixels (the zero padding and ragged tile edges) are filled with zeros by the TMA unit.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "conv_common.cuh"

namespace kxc_b200 {

enum TcDType : int { kTcBF16 = 0, kTcTF32 = 1, kTcS8 = 2 };

enum TcOutMode : int {
    kOutNHWC_BF16 = 0,  // activations for the next layer
    kOutNHWC_F32 = 1,   // fp32 activations / dense logits [M, Cout]
    kOutNCHW_F32 = 2,   // the reference's own tensor layout (per-op entry points)
    kOutNHWC_S8 = 3,    // requantized int8
    kOutNCHW_S8 = 4
};

struct alignas(64) TcParams {
    CUtensorMap tmA[4];  // stride 1: [0]; stride 2: one map per (row parity, column parity) of the input
    CUtensorMap tmB;
    int N, OH, OW, Cout;
    int taps_h, taps_w;          // filter taps walked by the K loop
    int stride;                  // 1 or 2 (same in h and w)
    int pad_h, pad_w, dil_h, dil_w;
    int cblocks;                 // channel blocks per tap
    int kb_elems;                // elements per K block (row of a stage)
    int BW, BH, BNI;             // tile box: cols x rows x images (BW*BH*BNI <= 128)
    int tiles_w, tiles_h, tiles_n, tiles_c;
    int relu;
    int round_out_tf32;          // kOutNHWC_F32 only: round stored values to tf32 (they feed another tf32 contraction)
    int vec_ok;                  // bias/residual/out (int8: bias/multiplier/shift/out) base pointers are 16-byte aligned: vector epilogue allowed
    const float* bias;           // fp32 bias (float paths), may be null
    const int32_t* bias_i32;     // int32 bias (int8 path)
    const int32_t* multiplier;   // int8 path
    const int32_t* shift;        // int8 path
    const void* residual;        // same layout/dtype as out, may be null
    void* out;
    int* status;                 // device status word; non-zero after a bounded wait ran out
    // direct stem kernel only (conv_stem.cu): packed input / core-matrix weights, packed row pitch, padded height
    const void* aux_in;
    const void* aux_w;
    int aux_row_bytes, aux_hp;
    // 1: work items are taken from the last to the first. A plan alternates the direction from launch to launch, so a
    // kernel starts on the images its producer wrote last, which are still in L2 (same items, same results).
    int reverse;
    int aux_c, aux_h, aux_w_px;  // fused-input stem kernel (conv_stem_fused.cu): channels, height, width of the NCHW fp32 input
    // second output of the dual kernel: a 1x1 convolution of the same stride over the same input (the residual
    // branch's downsample next to a block's first 3x3 stride-2 convolution); its reduction runs as extra K blocks
    // over the centre tap's pixels into a second accumulator
    CUtensorMap tmB2;
    const float* bias2;
    void* out2;
    int relu2;
    // TMA stores of the output (tc_bind_store): each epilogue warp's 32 pixels x 64 channels leave as one box
    CUtensorMap tmOut, tmOut2;
    int store_box;               // 1 when tmOut (and tmOut2 for the two-output form) are valid
};

struct TcConfig {
    TcDType dtype;
    int kb_bytes;  // 32, 64 or 128 (also the TMA/UMMA swizzle span)
    int bn;        // 64, 128 or 256
    TcOutMode out_mode;
    int ctas = 1;  // 2: clusters of two CTAs share each B tile (tcgen05 cta_group::2, M = 256 per instruction)
    int dual = 0;  // 1: also computes the 1x1 convolution described by tmB2 / bias2 / out2 / relu2
    int mt = 1;    // 2: two pixel tiles per work item share each B tile (two accumulate chains in flight)
};

// Sets vec_ok from the epilogue pointers; call after filling bias/residual/out.
inline void tc_finish_params(TcParams* p) {
    auto al = [](const void* q) { return q == nullptr || (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    p->vec_ok = al(p->bias) && al(p->residual) && al(p->out) && al(p->bias_i32) && al(p->multiplier) && al(p->shift) ? 1 : 0;
}

// Launches the persistent kernel for the given configuration. `p` must be fully populated.
int32_t tc_launch(const TcConfig& cfg, const TcParams& p, cudaStream_t stream);

// Tile box selection: maximise the fraction of the 128 rows that are real output pixels.
void tc_pick_tile(int N, int OH, int OW, int* BW, int* BH, int* BNI);

// Tensor map helpers (driver entry point resolved at run time; no link against libcuda).
int32_t tc_make_tmap(CUtensorMap* out, TcDType dtype, int rank, void* base, const uint64_t* dims,
                     const uint64_t* strides_bytes, const uint32_t* box, int swizzle_bytes);

// Device status word shared by all tensor-core launches of this process (lazily allocated, zeroed).
int32_t tc_status_word(int** out);

// conv_static_scratch.cu: the status word of the entry point that allocates nothing (nullptr until it has been
// used on the current device).
int32_t static_scratch_status_word(int** out);

// Fills tmA/tmB and the geometry of `p` for a regular convolution over an NHWC activation tensor
// with `cpad` channels and weights packed as [Cout][KH][KW][cpad].
// `status_word`: device int the kernel reports a run-out wait into; nullptr = the process-wide word
// from tc_status_word().
int32_t tc_setup_conv(TcParams* p, TcConfig* cfg, TcDType dtype, TcOutMode out_mode, const void* act_nhwc,
                      const void* w_packed, int N, int H, int W, int cpad, int Cout, int KH, int KW, int stride, int pad_h,
                      int pad_w, int dil_h, int dil_w, int* status_word = nullptr);

// Whether a KHxKW convolution (stride, padding, dilation as given) can carry a 1x1 convolution of the same stride
// and no padding as its second output, and the setup of that second output (call after tc_setup_conv, which it
// re-runs with the dual kernel's 128-wide tile).
bool tc_dual_applicable(TcDType dtype, TcOutMode out_mode, int cpad, int Cout, int KH, int KW, int stride, int pad_h, int pad_w,
                        int dil_h, int dil_w);
// After p->out (and p->out2) are final: builds the store maps when the configuration allows boxed stores (bf16 NHWC
// output, full 128-pixel tiles whose 32-pixel quarters are boxes of the output tensor, channel count a multiple of 64)
// and sets p->store_box; otherwise leaves the per-thread store path in place. KXC_B200_TMA_STORE=0 disables it.
int32_t tc_bind_store(TcParams* p, const TcConfig& cfg);
int32_t tc_setup_dual(TcParams* p, TcConfig* cfg, const void* act_nhwc, const void* w_packed, const void* w2_packed, int N,
                      int H, int W, int cpad, int Cout, int KH, int KW, int stride, int pad_h, int pad_w);

inline int tc_elem_bytes(TcDType t) { return t == kTcBF16 ? 2 : (t == kTcTF32 ? 4 : 1); }
// Channel padding the tensor-core path needs for `c` input channels: one K block per tap must be
// 32, 64 or a multiple of 128 bytes.
inline int tc_channel_pad(TcDType t, int c) {
    const int eb = tc_elem_bytes(t);
    const int e32 = 32 / eb, e64 = 64 / eb, e128 = 128 / eb;
    if (c <= e32) return e32;
    if (c <= e64) return e64;
    return (c + e128 - 1) / e128 * e128;
}

}  // namespace kxc_b200

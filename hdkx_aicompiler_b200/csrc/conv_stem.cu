// Direct stride-2 "stem" convolution (few input channels, KW <= 8, 64 output channels; the 7x7/s2
// first layer of ResNet) on tcgen05 + TMEM, bf16.
//
// Input: the packed stem layout [N][Hp][Wp][4] bf16 with a zero border (8 bytes per pixel). For output
// pixel (oh, ow) and filter row kh the K vector is the 8 consecutive pixels x 4 channels that start at
// packed pixel (2*oh + kh, 2*ow): 64 contiguous bytes, and the vector of ow+1 starts 16 bytes later.
// In the UNSWIZZLED K-major operand layout the rows of an 8-row core matrix are exactly 16 bytes apart
// and the two 16-byte K chunks of one MMA are `leading byte offset` apart, so with LBO = 16 and
// SBO = 128 the A operand of 128 consecutive output columns is simply a window of ONE packed input row
// in shared memory — overlapping rows, no im2col copy, no per-tap TMA box.
//
// A CTA owns a strip of R consecutive output rows of one image: the 2R+5 packed input rows it needs
// are fetched with one bulk copy (they are contiguous in global memory), each input row is used by up
// to four output rows, and the 28 KiB of weights stay resident in shared memory in core-matrix order
// [kh][k-chunk][cout][8]. Per output row: KH x 2 MMAs (M = 128 columns, N = 64, K = 16).
//
// Roles as in conv_tc.cu (producer warp, MMA warp + TMEM owner, 8 epilogue warps, two accumulators,
// bounded waits).
#include "conv_stem.cuh"

#include <climits>

#include <cuda_bf16.h>

#include <cmath>
#include <mutex>

#include "common.cuh"
#include "conv_epilogue.cuh"
#include "sm100.cuh"

namespace kxc_b200 {
namespace {

using namespace sm100;

constexpr int kThreads = 320;
constexpr int kBN = 64;
constexpr int kMaxKH = 7;
constexpr int kStripRows = 8;                         // output rows per strip
constexpr int kMaxInRows = 2 * (kStripRows - 1) + kMaxKH;  // 21
constexpr int kMaxRowBytes = 2048;                    // packed row (Wp * 8 bytes) upper bound
constexpr int kStripBytes = ((kMaxInRows * kMaxRowBytes + 4096 + 1023) / 1024) * 1024;  // + slack for the M=128 over-read
constexpr int kStages = 3;
constexpr int kWeightBytes = kMaxKH * 4 * kBN * 16;   // 28672
constexpr int kSmemBytes = kWeightBytes + kStages * kStripBytes + 1024;

// Descriptors: unswizzled K-major — rows 16 B apart inside a core matrix (fixed by the layout), K chunks
// `leading byte offset` apart (16 B for the overlapping input rows, 1024 B for the weights), 8-row groups 128 B apart.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}

// kKind = F16: packed bf16 pixels [4 channels], bf16 NHWC output. kKind = I8: packed int8 pixels [8 channels] (the same
// 8 bytes per pixel, so every address below is unchanged; one instruction covers K = 32 bytes either way), int32
// accumulators, fixed-point requantize to int8 in the output layout kOutMode.
template <MmaKind kKind, int kOutMode>
__global__ void __launch_bounds__(kThreads, 1) conv_stem_direct_kernel(const __grid_constant__ TcParams p) {
    constexpr uint32_t kTmemCols = 2 * kBN;
    constexpr uint32_t kIdesc = kKind == MmaKind::I8 ? make_instr_desc(kFmtS8, kAccS32, kBN) : make_instr_desc(kFmtBF16, kAccF32, kBN);

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_w;
    __shared__ __align__(8) uint64_t bar_full[kStages];
    __shared__ __align__(8) uint64_t bar_empty[kStages];
    __shared__ __align__(8) uint64_t bar_acc_full[2];
    __shared__ __align__(8) uint64_t bar_acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    // int8: per output channel the constants of the high-word requantize (requant_prepare), prepared once per CTA;
    // q_fast = 0 when some channel does not qualify (the general formula is used then)
    __shared__ __align__(16) int4 q_tab[kKind == MmaKind::I8 ? kBN : 1];
    __shared__ int q_fast;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t w_smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t strip_smem = w_smem + kWeightBytes;

    const int KH = p.taps_h;
    if constexpr (kKind == MmaKind::I8) {
        if (threadIdx.x == 0) q_fast = 1;
        __syncthreads();
        // |accumulator| <= 128 * 128 * (KH rows * 8 columns * 8 channels); the constants are call arguments
        if (threadIdx.x >= 64 && threadIdx.x < 64 + kBN) {
            const int c = threadIdx.x - 64;
            if (!requant_prepare(__ldg(p.bias_i32 + c), __ldg(p.multiplier + c), __ldg(p.shift + c), 128ll * 128 * 64 * KH, &q_tab[c]))
                q_fast = 0;
        }
    }
    const int row_bytes = p.aux_row_bytes;          // Wp * 8
    const int Hp = p.aux_hp;
    const int strips_per_image = (p.OH + kStripRows - 1) / kStripRows;
    const int total_strips = strips_per_image * p.N;
    const uint8_t* in_base = static_cast<const uint8_t*>(p.aux_in);

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar_w), 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bar_acc_full[a]), 1);
            mbar_init(smem_u32(&bar_acc_empty[a]), 8);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
        tmem_relinquish();
    }
    // The MMA of the last output columns reads a little past the last copied input row: make sure those
    // bytes are finite bf16 (they only feed accumulator rows that are never stored).
    for (uint32_t i = threadIdx.x; i < (uint32_t)(kStages * kStripBytes / 16); i += kThreads) {
        const uint32_t addr = strip_smem + i * 16;
        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int* abort_ptr = &abort_flag;
    pdl_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t wbytes = (uint32_t)(KH * 4 * kBN * 16);
            mbar_arrive_expect_tx(smem_u32(&bar_w), wbytes);
            bulk_copy_g2s(w_smem, p.aux_w, wbytes, smem_u32(&bar_w));  // constants: no need to wait for the previous kernel
            pdl_wait();
            int stage = 0;
            uint32_t phase = 0;
            for (int strip = blockIdx.x; strip < total_strips; strip += gridDim.x) {
                const int n = strip / strips_per_image;
                const int oh0 = (strip - n * strips_per_image) * kStripRows;
                const int rows_out = (p.OH - oh0) < kStripRows ? (p.OH - oh0) : kStripRows;
                int rows_in = 2 * (rows_out - 1) + KH;
                if (2 * oh0 + rows_in > Hp) rows_in = Hp - 2 * oh0;
                if (!mbar_wait_bounded(smem_u32(&bar_empty[stage]), phase ^ 1u, abort_ptr)) break;
                const uint32_t full = smem_u32(&bar_full[stage]);
                const uint32_t bytes = (uint32_t)(rows_in * row_bytes);
                mbar_arrive_expect_tx(full, bytes);
                bulk_copy_g2s(strip_smem + stage * kStripBytes, in_base + ((size_t)n * Hp + 2 * oh0) * row_bytes, bytes, full);
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = mbar_wait_bounded(smem_u32(&bar_w), 0, abort_ptr);
            const uint32_t ab_hi = desc_hi(128, 0);  // unswizzled, 8-row groups 128 B apart (A and B alike)
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            for (int strip = blockIdx.x; ok && strip < total_strips; strip += gridDim.x) {
                const int oh0 = (strip % strips_per_image) * kStripRows;
                const int rows_out = (p.OH - oh0) < kStripRows ? (p.OH - oh0) : kStripRows;
                if (!mbar_wait_bounded(smem_u32(&bar_full[stage]), phase, abort_ptr)) break;
                tc_fence_after_sync();
                const uint32_t strip_base = strip_smem + stage * kStripBytes;
                for (int rr = 0; rr < rows_out; ++rr) {
                    if (!mbar_wait_bounded(smem_u32(&bar_acc_empty[acc]), acc_phase ^ 1u, abort_ptr)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + (uint32_t)(acc * kBN);
                    uint32_t a_lo = desc_lo(strip_base + (uint32_t)(2 * rr * row_bytes), 16);
                    uint32_t b_lo = desc_lo(w_smem, kBN * 16);
                    for (int kh = 0; kh < KH; ++kh) {
                        if constexpr (kKind == MmaKind::I8) {
                            umma_i8_split(d_tmem, a_lo, ab_hi, b_lo, ab_hi, kIdesc, kh != 0 ? 1u : 0u);
                            umma_i8_split(d_tmem, a_lo + 2u, ab_hi, b_lo + (uint32_t)((2 * kBN * 16) >> 4), ab_hi, kIdesc, 1u);
                        } else {
                            umma_f16_split(d_tmem, a_lo, ab_hi, b_lo, ab_hi, kIdesc, kh != 0 ? 1u : 0u);
                            umma_f16_split(d_tmem, a_lo + 2u, ab_hi, b_lo + (uint32_t)((2 * kBN * 16) >> 4), ab_hi, kIdesc, 1u);
                        }
                        a_lo += (uint32_t)(row_bytes >> 4);
                        b_lo += (uint32_t)((4 * kBN * 16) >> 4);
                    }
                    umma_commit(smem_u32(&bar_acc_full[acc]));
                    acc ^= 1;
                    if (acc == 0) acc_phase ^= 1u;
                }
                if (!ok) break;
                umma_commit(smem_u32(&bar_empty[stage]));
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
        }
    } else {
        const int quad = warp & 3;
        const int half = (warp - 2) >> 2;
        const int ow = quad * 32 + lane;
        const int c0 = half * 32;
        const bool col_ok = ow < p.OW;
        pdl_wait();
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int strip = blockIdx.x; ok && strip < total_strips; strip += gridDim.x) {
            const int n = strip / strips_per_image;
            const int oh0 = (strip - n * strips_per_image) * kStripRows;
            const int rows_out = (p.OH - oh0) < kStripRows ? (p.OH - oh0) : kStripRows;
            for (int rr = 0; rr < rows_out; ++rr) {
                ok = mbar_wait_bounded(smem_u32(&bar_acc_full[acc]), acc_phase, abort_ptr);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after_sync();
                uint32_t v[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * kBN + c0), v);
                tmem_ld_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[acc]));
                if constexpr (kKind == MmaKind::I8) {
                    if (q_fast && p.vec_ok) {
                        if (col_ok) {
                            const int32_t lo = p.relu ? 0 : INT32_MIN;
                            uint32_t qw[8];
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                const uint32_t vv[4] = {v[j], v[j + 1], v[j + 2], v[j + 3]};
                                const int4 qq[4] = {q_tab[c0 + j], q_tab[c0 + j + 1], q_tab[c0 + j + 2], q_tab[c0 + j + 3]};  // broadcasts
                                qw[j >> 2] = requant4_prepared(vv, qq, lo);
                            }
                            int8_t* out = static_cast<int8_t*>(p.out);
                            if constexpr (kOutMode == kOutNHWC_S8) {
                                uint4* dst = reinterpret_cast<uint4*>(out + (((size_t)n * p.OH + (oh0 + rr)) * p.OW + ow) * kBN + c0);
                                dst[0] = make_uint4(qw[0], qw[1], qw[2], qw[3]);
                                dst[1] = make_uint4(qw[4], qw[5], qw[6], qw[7]);
                            } else {  // NCHW: consecutive lanes are consecutive columns, a channel's store is one 32-byte run
                                const size_t plane = (size_t)p.OH * p.OW;
                                int8_t* dst = out + ((size_t)n * kBN + c0) * plane + (size_t)(oh0 + rr) * p.OW + ow;
#pragma unroll
                                for (int j = 0; j < 32; ++j) dst[(size_t)j * plane] = (int8_t)(qw[j >> 2] >> (8 * (j & 3)));
                            }
                        }
                    } else {
                        epilogue_chunk<kOutMode>(p, v, c0, col_ok, n, oh0 + rr, ow);
                    }
                } else if (col_ok) {
                    const size_t pix = ((size_t)n * p.OH + (oh0 + rr)) * p.OW + ow;
                    const uint4 no_res[4] = {};
                    epilogue_fast_bf16(p, v, c0, pix, no_res, false);
                }
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
    }

    if (*abort_ptr) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc(tmem_base, kTmemCols);
    }
    if (threadIdx.x == 0 && *abort_ptr && p.status != nullptr) atomicExch(p.status, KXC_B200_ERR_DEVICE_WAIT);
}

// ------------------------------------------------------------------------------------------------------
// Stem convolution + bias + ReLU + max_pool2d(3x3, stride 2, pad 1) in one kernel.
//
// The convolution's output (the largest activation of the network) never goes to HBM, nor to shared memory: an
// epilogue thread holds one conv pixel's 32 channels as 16 packed bf16 pairs (after bias, ReLU and rounding, i.e.
// exactly the values the unfused kernel would store) and pools in registers. Horizontally the window of pooled
// column pw is conv columns 2pw-1, 2pw, 2pw+1: the thread of the even column takes its neighbours' values with
// two warp shuffles per register (the one neighbour that lives in another warp, the left one of a warp's first
// column, comes through a 64-byte shared-memory slot). Vertically the three conv rows of a pooled row arrive one
// after the other, so a running maximum suffices. A strip is 9 conv rows (8s-1 .. 8s+7; the first one is
// recomputed from the strip above) = 4 pooled rows.
// After ReLU no value is NaN (NaN > 0 is false, so ReLU maps it to +0), negative or -0. On such values the
// reference's fold `m = (m > v) ? m : v` from -inf, with -1e30 for padding, is exactly the numeric maximum of the
// in-bounds taps in any order, and 0 is a neutral element: packed bf16 max instructions give the identical bits
// as conv kernel + pool kernel.
constexpr int kPoolStages = 3;
constexpr int kPoolConvRows = kStripRows + 1;                          // 9 conv rows per strip
constexpr int kPoolInRows = 2 * (kPoolConvRows - 1) + kMaxKH;          // 23 packed input rows
constexpr int kPoolStripBytes = ((kPoolInRows * kMaxRowBytes + 4096 + 1023) / 1024) * 1024;
constexpr int kExchBytes = 2 * 2 * 4 * 64;  // [row parity][channel half][quadrant] x 64 bytes: a warp's last column
constexpr int kPoolSmemBytes = kWeightBytes + kPoolStages * kPoolStripBytes + kExchBytes + 1024;

__global__ void __launch_bounds__(kThreads, 1) conv_stem_pool_kernel(const __grid_constant__ TcParams p) {
    // conv rows whose MMAs are interleaved (independent accumulate chains); measured: 2 -> 0.78 ms, 4 -> 0.86 ms
    constexpr int kFlight = 2;
    constexpr int kPAccs = 2 * kFlight;      // accumulators: kFlight on the tensor core + kFlight being drained
    constexpr uint32_t kTmemCols = kPAccs * kBN;
    constexpr uint32_t kIdesc = make_instr_desc(kFmtBF16, kAccF32, kBN);

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_w;
    __shared__ __align__(8) uint64_t bar_full[kPoolStages];
    __shared__ __align__(8) uint64_t bar_empty[kPoolStages];
    __shared__ __align__(8) uint64_t bar_acc_full[kPAccs];
    __shared__ __align__(8) uint64_t bar_acc_empty[kPAccs];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t w_smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t strip_smem = w_smem + kWeightBytes;
    const uint32_t exch_smem = strip_smem + kPoolStages * kPoolStripBytes;

    const int KH = p.taps_h;
    const int row_bytes = p.aux_row_bytes;
    const int Hp = p.aux_hp;
    const int strips_per_image = p.OH / kStripRows;  // OH is a multiple of 8 for this kernel
    const int total_strips = strips_per_image * p.N;
    const uint8_t* in_base = static_cast<const uint8_t*>(p.aux_in);

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar_w), 1);
        for (int s = 0; s < kPoolStages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int a = 0; a < kPAccs; ++a) {
            mbar_init(smem_u32(&bar_acc_full[a]), 1);
            mbar_init(smem_u32(&bar_acc_empty[a]), 8);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
        tmem_relinquish();
    }
    for (uint32_t i = threadIdx.x; i < (uint32_t)(kPoolStages * kPoolStripBytes / 16); i += kThreads) {
        const uint32_t addr = strip_smem + i * 16;
        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int* abort_ptr = &abort_flag;
    pdl_launch_dependents();

    // Strip s of an image covers conv rows 8s-1 .. 8s+7 (local j = 0..8; j = 0 is skipped for s = 0, it is the
    // pool's padding row) and packed input rows from max(16s-2, 0).
    if (warp == 0) {
        if (lane == 0) {
            const uint32_t wbytes = (uint32_t)(KH * 4 * kBN * 16);
            mbar_arrive_expect_tx(smem_u32(&bar_w), wbytes);
            bulk_copy_g2s(w_smem, p.aux_w, wbytes, smem_u32(&bar_w));  // constants: no need to wait for the previous kernel
            pdl_wait();
            int stage = 0;
            uint32_t phase = 0;
            for (int strip = blockIdx.x; strip < total_strips; strip += gridDim.x) {
                const int n = strip / strips_per_image;
                const int s = strip - n * strips_per_image;
                const int row0 = s > 0 ? 16 * s - 2 : 0;
                int rows_in = (s > 0 ? 2 * (kPoolConvRows - 1) : 2 * (kPoolConvRows - 2)) + KH;
                if (row0 + rows_in > Hp) rows_in = Hp - row0;
                if (!mbar_wait_bounded(smem_u32(&bar_empty[stage]), phase ^ 1u, abort_ptr)) break;
                const uint32_t full = smem_u32(&bar_full[stage]);
                const uint32_t bytes = (uint32_t)(rows_in * row_bytes);
                mbar_arrive_expect_tx(full, bytes);
                bulk_copy_g2s(strip_smem + stage * kPoolStripBytes, in_base + ((size_t)n * Hp + row0) * row_bytes, bytes, full);
                if (++stage == kPoolStages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = mbar_wait_bounded(smem_u32(&bar_w), 0, abort_ptr);
            const uint32_t ab_hi = desc_hi(128, 0);  // unswizzled, 8-row groups 128 B apart (A and B alike)
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            for (int strip = blockIdx.x; ok && strip < total_strips; strip += gridDim.x) {
                const int s = strip % strips_per_image;
                if (!mbar_wait_bounded(smem_u32(&bar_full[stage]), phase, abort_ptr)) break;
                tc_fence_after_sync();
                const uint32_t strip_base = strip_smem + stage * kPoolStripBytes;
                // kFlight conv rows at a time, their MMAs alternating between as many accumulators: consecutive MMAs into
                // one accumulator are a dependent chain whose latency, not the tensor pipe, would otherwise set the pace
                for (int j = (s > 0 ? 0 : 1); j < kPoolConvRows; j += kFlight) {
                    const int rows = kPoolConvRows - j < kFlight ? kPoolConvRows - j : kFlight;
                    uint32_t d[kFlight];
#pragma unroll
                    for (int u = 0; u < kFlight; ++u) {
                        if (u < rows) {
                            const int a = (acc + u) & (kPAccs - 1);
                            const uint32_t ph = (acc + u) >= kPAccs ? acc_phase ^ 1u : acc_phase;
                            if (ok && !mbar_wait_bounded(smem_u32(&bar_acc_empty[a]), ph ^ 1u, abort_ptr)) ok = false;
                            d[u] = tmem_base + (uint32_t)(a * kBN);
                        }
                    }
                    if (!ok) break;
                    tc_fence_after_sync();
                    const int in_row0 = s > 0 ? 2 * j : 2 * j - 2;  // local packed row of filter row 0 of conv row j
                    uint32_t a_lo = desc_lo(strip_base + (uint32_t)(in_row0 * row_bytes), 16);
                    const uint32_t next_row = (uint32_t)((2 * row_bytes) >> 4);  // the next conv row starts two packed rows lower
                    uint32_t b_lo = desc_lo(w_smem, kBN * 16);
                    for (int kh = 0; kh < KH; ++kh) {
                        const uint32_t accum = kh != 0 ? 1u : 0u;
#pragma unroll
                        for (int u = 0; u < kFlight; ++u)
                            if (u < rows) umma_f16_split(d[u], a_lo + (uint32_t)u * next_row, ab_hi, b_lo, ab_hi, kIdesc, accum);
#pragma unroll
                        for (int u = 0; u < kFlight; ++u)
                            if (u < rows)
                                umma_f16_split(d[u], a_lo + (uint32_t)u * next_row + 2u, ab_hi, b_lo + (uint32_t)((2 * kBN * 16) >> 4), ab_hi,
                                               kIdesc, 1u);
                        a_lo += (uint32_t)(row_bytes >> 4);
                        b_lo += (uint32_t)((4 * kBN * 16) >> 4);
                    }
                    for (int u = 0; u < rows; ++u) {
                        umma_commit(smem_u32(&bar_acc_full[acc]));
                        acc = (acc + 1) & (kPAccs - 1);
                        if (acc == 0) acc_phase ^= 1u;
                    }
                }
                if (!ok) break;
                umma_commit(smem_u32(&bar_empty[stage]));
                if (++stage == kPoolStages) { stage = 0; phase ^= 1u; }
            }
        }
    } else {
        const int quad = warp & 3;
        const int half = (warp - 2) >> 2;
        const int ow = quad * 32 + lane;
        const int c0 = half * 32;
        const int POH = p.OH / 2, POW = p.OW / 2;
        __nv_bfloat16* pooled = static_cast<__nv_bfloat16*>(p.out);
        const bool centre = (lane & 1) == 0 && ow < p.OW;  // even conv columns are the pooling windows' centres
        float bias[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) bias[e] = p.bias != nullptr ? __ldg(p.bias + c0 + e) : 0.0f;
        pdl_wait();
        int acc = 0;
        uint32_t acc_phase = 0;
        uint32_t row_ctr = 0;  // conv rows handled so far (parity picks the exchange slot)
        bool ok = true;
        for (int strip = blockIdx.x; ok && strip < total_strips; strip += gridDim.x) {
            const int n = strip / strips_per_image;
            const int s = strip - n * strips_per_image;
            uint32_t vmax[16];  // running maximum over the conv rows of the current pooled row (0 is neutral)
#pragma unroll
            for (int e = 0; e < 16; ++e) vmax[e] = 0u;
            for (int j = (s > 0 ? 0 : 1); j < kPoolConvRows; ++j, ++row_ctr) {
                // A wait that runs out must not leave some warps behind at the barrier below: the failure is carried
                // to the barrier, where the four warps of this channel half learn of it and leave together.
                bool bad = !__all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&bar_acc_full[acc]), acc_phase, abort_ptr));
                uint32_t pk[16];
                if (!bad) {
                    tc_fence_after_sync();
                    uint32_t v[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * kBN + c0), v);
                    tmem_ld_wait();
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[acc]));
                    acc = (acc + 1) & (kPAccs - 1);
                    if (acc == 0) acc_phase ^= 1u;
                    // +bias, ReLU, round to bf16: the values the unfused convolution kernel stores
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        float a = __fadd_rn(__uint_as_float(v[2 * e]), bias[2 * e]);
                        float b = __fadd_rn(__uint_as_float(v[2 * e + 1]), bias[2 * e + 1]);
                        if (p.relu) {
                            a = a > 0.0f ? a : 0.0f;
                            b = b > 0.0f ? b : 0.0f;
                        }
                        pk[e] = pack_bf16(a, b);
                    }
                    if (ow >= p.OW) {  // columns beyond the image (the M = 128 tile is wider) must not win a maximum
#pragma unroll
                        for (int e = 0; e < 16; ++e) pk[e] = 0u;
                    }
                    if (lane == 31) {  // the left neighbour of the next quadrant's first column
                        const uint32_t slot = exch_smem + ((((row_ctr & 1u) * 2u + (uint32_t)half) * 4u + (uint32_t)quad) * 64u);
#pragma unroll
                        for (int g = 0; g < 4; ++g)
                            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(slot + g * 16u), "r"(pk[4 * g]), "r"(pk[4 * g + 1]),
                                         "r"(pk[4 * g + 2]), "r"(pk[4 * g + 3])
                                         : "memory");
                    }
                }
                if (named_barrier_or(1 + half, 128, bad)) {
                    ok = false;
                    break;
                }
                // horizontal maximum over columns ow-1, ow, ow+1 (meaningful in the centre threads)
                uint32_t left[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) left[e] = __shfl_up_sync(0xffffffffu, pk[e], 1);
                if (lane == 0) {
                    if (quad == 0) {
#pragma unroll
                        for (int e = 0; e < 16; ++e) left[e] = 0u;  // column -1 is padding
                    } else {
                        const uint32_t slot = exch_smem + ((((row_ctr & 1u) * 2u + (uint32_t)half) * 4u + (uint32_t)(quad - 1)) * 64u);
#pragma unroll
                        for (int g = 0; g < 4; ++g)
                            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                         : "=r"(left[4 * g]), "=r"(left[4 * g + 1]), "=r"(left[4 * g + 2]), "=r"(left[4 * g + 3])
                                         : "r"(slot + g * 16u));
                    }
                }
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const uint32_t right = __shfl_down_sync(0xffffffffu, pk[e], 1);
                    __nv_bfloat162 m = __hmax2(*reinterpret_cast<__nv_bfloat162*>(&left[e]), *reinterpret_cast<__nv_bfloat162*>(&pk[e]));
                    m = __hmax2(m, *reinterpret_cast<const __nv_bfloat162*>(&right));
                    left[e] = *reinterpret_cast<uint32_t*>(&m);  // this row's horizontal maximum
                    m = __hmax2(m, *reinterpret_cast<__nv_bfloat162*>(&vmax[e]));
                    vmax[e] = *reinterpret_cast<uint32_t*>(&m);
                }
                // local rows 0, 2, 4, 6, 8 are conv rows 8s-1, 8s+1, ...: the last row of one pooled row and the first
                // of the next
                if ((j & 1) == 0) {
                    if (j >= 2 && centre) {
                        const int ph = 4 * s + j / 2 - 1;
                        uint4* dst = reinterpret_cast<uint4*>(pooled + ((((size_t)n * POH + ph) * POW + (ow >> 1)) * kBN) + c0);
#pragma unroll
                        for (int g = 0; g < 4; ++g) dst[g] = make_uint4(vmax[4 * g], vmax[4 * g + 1], vmax[4 * g + 2], vmax[4 * g + 3]);
                    }
#pragma unroll
                    for (int e = 0; e < 16; ++e) vmax[e] = left[e];  // the running maximum restarts with this row
                }
            }
        }
    }

    if (*abort_ptr) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc(tmem_base, kTmemCols);
    }
    if (threadIdx.x == 0 && *abort_ptr && p.status != nullptr) atomicExch(p.status, KXC_B200_ERR_DEVICE_WAIT);
}

// Stem weights in core-matrix order: [KH][4 k-chunks][64 cout][8] bf16, element e of chunk j = pixel 2j + e/4,
// channel e%4; zero for kw >= KW or c >= C.
__global__ void stem_pack_weights_core_kernel(const float* __restrict__ w, __nv_bfloat16* __restrict__ out, int O, int C,
                                              int KH, int KW) {
    const int total = KH * 4 * kBN * 8;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int e = i & 7, o = (i >> 3) & (kBN - 1), j = (i >> 9) & 3, kh = i >> 11;
        const int kw = 2 * j + (e >> 2), c = e & 3;
        float f = 0.0f;
        if (o < O && c < C && kw < KW) f = w[((o * C + c) * KH + kh) * KW + kw];
        out[i] = __float2bfloat16_rn(f);
    }
}

// int8 stem: NCHW int8 [N,C<=8,H,W] -> packed [N][Hp][Wp][8] int8 with a zero border (8 bytes per pixel)
// (kNhwcIn: the input is [N,H,W,C] instead of [N,C,H,W])
template <bool kNhwcIn>
__global__ void __launch_bounds__(256) stem_pack_s8_kernel(const int8_t* __restrict__ x, uint2* __restrict__ out, int N, int C, int H,
                                                            int W, int Hp, int Wp, int pad_h, int pad_w) {
    const int64_t total = (int64_t)N * Hp * Wp;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
        const int wp = (int)(i % Wp);
        int64_t t = i / Wp;
        const int hp = (int)(t % Hp);
        const int n = (int)(t / Hp);
        const int h = hp - pad_h, w = wp - pad_w;
        uint32_t lo = 0, hi = 0;
        if (h >= 0 && h < H && w >= 0 && w < W) {
            for (int c = 0; c < C; ++c) {
                const uint32_t b = kNhwcIn ? (uint8_t)__ldg(x + (((int64_t)n * H + h) * W + w) * C + c)
                                           : (uint8_t)__ldg(x + (((int64_t)n * C + c) * H + h) * W + w);
                if (c < 4) lo |= b << (8 * c);
                else hi |= b << (8 * (c - 4));
            }
        }
        out[i] = make_uint2(lo, hi);
    }
}

// int8 stem weights in core-matrix order: [KH][4 k-chunks][64 cout][16 bytes]; byte e of chunk j = pixel 2j + e/8,
// channel e%8; zero for kw >= KW or c >= C.
// (kOhwi: the weights are [O,KH,KW,C] instead of [O,C,KH,KW])
template <bool kOhwi>
__global__ void stem_pack_weights_core_s8_kernel(const int8_t* __restrict__ w, int8_t* __restrict__ out, int O, int C, int KH, int KW) {
    const int total = KH * 4 * kBN * 16;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int e = i & 15, o = (i >> 4) & (kBN - 1), j = (i >> 10) & 3, kh = i >> 12;
        const int kw = 2 * j + (e >> 3), c = e & 7;
        int8_t v = 0;
        if (o < O && c < C && kw < KW) v = kOhwi ? w[((o * KH + kh) * KW + kw) * C + c] : w[((o * C + c) * KH + kh) * KW + kw];
        out[i] = v;
    }
}

}  // namespace

bool stem_direct_s8_applicable(int C, int O, int KH, int KW, int stride, int dil, int W, int OW, int Wp) {
    return C <= 8 && O == kBN && KH <= kMaxKH && KW <= 8 && stride == 2 && dil == 1 && W >= 8 && OW <= 128 && Wp * 8 <= kMaxRowBytes &&
           (Wp * 8) % 16 == 0;
}

int32_t stem_direct_s8_pack(const int8_t* x, const int8_t* w, void* packed_x, void* packed_w, int N, int C, int H, int W, int O, int KH,
                            int KW, int Hp, int Wp, int pad_h, int pad_w, bool nhwc, cudaStream_t s) {
    const int64_t total = (int64_t)N * Hp * Wp;
    int64_t blocks = (total + 255) / 256;
    if (blocks > (int64_t)kNumSMs * 16) blocks = (int64_t)kNumSMs * 16;
    const int wblocks = (KH * 4 * kBN * 16 + 255) / 256;
    if (nhwc) {
        stem_pack_s8_kernel<true><<<(int)blocks, 256, 0, s>>>(x, static_cast<uint2*>(packed_x), N, C, H, W, Hp, Wp, pad_h, pad_w);
        KXC_TRY(check_launch("stem_pack_s8"));
        stem_pack_weights_core_s8_kernel<true><<<wblocks, 256, 0, s>>>(w, static_cast<int8_t*>(packed_w), O, C, KH, KW);
    } else {
        stem_pack_s8_kernel<false><<<(int)blocks, 256, 0, s>>>(x, static_cast<uint2*>(packed_x), N, C, H, W, Hp, Wp, pad_h, pad_w);
        KXC_TRY(check_launch("stem_pack_s8"));
        stem_pack_weights_core_s8_kernel<false><<<wblocks, 256, 0, s>>>(w, static_cast<int8_t*>(packed_w), O, C, KH, KW);
    }
    return check_launch("stem_pack_weights_core_s8");
}

template <MmaKind kKind, int kOutMode>
static int32_t stem_direct_launch_as(const TcParams& p, cudaStream_t stream) {
    static PerDeviceOnce smem_once;
    auto kernel = conv_stem_direct_kernel<kKind, kOutMode>;
    KXC_TRY(smem_opt_in(smem_once, kernel, kSmemBytes));
    const long long strips = (long long)((p.OH + kStripRows - 1) / kStripRows) * p.N;
    if (strips <= 0) return KXC_B200_OK;
    const int grid = (int)(strips < kNumSMs ? strips : kNumSMs);
    KXC_CUDA_TRY(launch_kernel(kernel, dim3(grid), dim3(kThreads), kSmemBytes, stream, /*pdl=*/true, 1, p));
    return check_launch("conv_stem_direct_kernel");
}

int32_t stem_direct_s8_launch(const TcParams& p, bool nhwc_out, cudaStream_t stream) {
    if (p.out == nullptr || p.bias_i32 == nullptr || p.multiplier == nullptr || p.shift == nullptr)
        return fail(KXC_B200_ERR_INVALID, "int8 stem conv: missing tensors");
    return nhwc_out ? stem_direct_launch_as<MmaKind::I8, kOutNHWC_S8>(p, stream) : stem_direct_launch_as<MmaKind::I8, kOutNCHW_S8>(p, stream);
}

bool stem_direct_applicable(TcDType dtype, int C, int O, int KH, int KW, int OW, int Wp) {
    return dtype == kTcBF16 && C <= 4 && O == kBN && KH <= kMaxKH && KW <= 8 && OW <= 128 && Wp * 8 <= kMaxRowBytes &&
           (Wp * 8) % 16 == 0;
}

size_t stem_direct_weight_bytes(int KH) { return (size_t)KH * 4 * kBN * 16; }

int32_t stem_direct_pack_weights(const float* w, void* out, int O, int C, int KH, int KW, cudaStream_t s) {
    stem_pack_weights_core_kernel<<<(KH * 4 * kBN * 8 + 255) / 256, 256, 0, s>>>(w, static_cast<__nv_bfloat16*>(out), O, C, KH, KW);
    return check_launch("stem_pack_weights_core");
}

int32_t stem_direct_setup(TcParams* p, const void* packed_in, const void* packed_w, int N, int OH, int OW, int KH, int Hp, int Wp) {
    p->N = N; p->OH = OH; p->OW = OW; p->Cout = kBN;
    p->taps_h = KH; p->taps_w = 1; p->stride = 2;
    p->BW = 128; p->BH = 1; p->BNI = 1;
    p->tiles_w = 1; p->tiles_h = OH; p->tiles_n = N; p->tiles_c = 1;
    p->aux_in = packed_in;
    p->aux_w = packed_w;
    p->aux_row_bytes = Wp * 8;
    p->aux_hp = Hp;
    KXC_TRY(tc_status_word(&p->status));
    return KXC_B200_OK;
}

bool stem_pool_applicable(int OH, int OW, int pool_k, int pool_s, int pool_pad) {
    return pool_k == 3 && pool_s == 2 && pool_pad == 1 && (OH % kStripRows) == 0 && (OW % 2) == 0 && OW <= 128;
}

int32_t stem_pool_launch(const TcParams& p, cudaStream_t stream) {
    static PerDeviceOnce smem_once;
    KXC_TRY(smem_opt_in(smem_once, conv_stem_pool_kernel, kPoolSmemBytes));
    if (!p.vec_ok || p.out == nullptr) return fail(KXC_B200_ERR_INVALID, "fused stem conv + pool: pointers must be 16-byte aligned");
    if (!p.relu) return fail(KXC_B200_ERR_INVALID, "fused stem conv + pool: the pooling shortcut relies on the ReLU in between");
    const long long strips = (long long)(p.OH / kStripRows) * p.N;
    if (strips <= 0) return KXC_B200_OK;
    const int grid = (int)(strips < kNumSMs ? strips : kNumSMs);
    KXC_CUDA_TRY(launch_kernel(conv_stem_pool_kernel, dim3(grid), dim3(kThreads), kPoolSmemBytes, stream, /*pdl=*/true, 1, p));
    return check_launch("conv_stem_pool_kernel");
}

int32_t stem_direct_launch(const TcParams& p, cudaStream_t stream) {
    if (!p.vec_ok || p.out == nullptr) return fail(KXC_B200_ERR_INVALID, "direct stem conv: pointers must be 16-byte aligned");
    return stem_direct_launch_as<MmaKind::F16, kOutNHWC_BF16>(p, stream);
}

}  // namespace kxc_b200

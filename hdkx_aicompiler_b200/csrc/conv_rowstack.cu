// 3x3 / stride-1 / pad-1 convolution for 64 -> 64 channel layers (bf16 NHWC) with the three filter ROWS stacked along
// the MMA's N dimension, on tcgen05 + TMEM.
//
// A tcgen05.mma fetches its A operand (128 pixels x 32 bytes) and its B operand (N x 32 bytes) from shared memory for
// every instruction, at roughly 64 bytes per clock, so with only 64 output channels (N = 64) an instruction spends
// ~96 cycles fetching for 32 cycles of math and two thirds of what it fetches is the A tile. Here one instruction
// multiplies the A tile with the weights of THREE taps at once:
//
//     D_r[i, w] = sum_kw W(r, kw) . X[i, w + kw - 1]        r = 0, 1, 2 (filter row), i = input row
//     out[oh, ow] = D_0[oh - 1, ow] + D_1[oh, ow] + D_2[oh + 1, ow]
//
// For a fixed kw the three D_r share the A operand X[i, w + kw - 1], so B = [W(0,kw); W(1,kw); W(2,kw)] (192 rows) and
// the accumulator holds D_0 | D_1 | D_2 in 192 TMEM columns: 12 instructions of N = 192 per tile instead of 36 of
// N = 64, i.e. 12 x 10 KB instead of 36 x 6 KB of operand fetch. The sum over r is taken in the epilogue, where it
// is a shift by one accumulator ROW: the tile's pixels are ordered column-major (TMEM lane = 16 * column + row), so
// rows i - 1 and i + 1 of the same column are the neighbouring lanes of the same warp (two warp shuffles per value).
//
//   * tile: 16 input rows x 8 columns -> 14 output rows x 8 columns; the input box is 16 rows x 10 columns x 64
//     channels, ONE TMA box per tile (20 KiB, zero-filled outside the image), stored [column][row][channel] by a
//     tensor map whose row dimension comes before its column dimension; the A operand of tap column kw is the
//     contiguous 128-pixel block that starts at column kw (a 2 KiB, swizzle-atom aligned offset);
//   * the 72 KiB of weights stay resident, ordered [kw][r][cout][cin] by nine TMA loads of the ordinary packed tensor.
//
// Roles as in conv_tc.cu: warp 0 producer, warp 1 MMA issuer + TMEM owner, warps 2..17 epilogue (two sets); two TMEM
// accumulators (the epilogue of one tile overlaps the next tile's MMAs); every wait bounded.
#include "conv_rowstack.cuh"

#include <climits>
#include <mutex>

#include "common.cuh"
#include "conv_epilogue.cuh"
#include "sm100.cuh"

namespace kxc_b200 {
namespace {

using namespace sm100;

// Two sets of eight epilogue warps, one per accumulator: set s drains the CTA's tiles of parity s, so the epilogues of
// consecutive tiles (three TMEM loads, 64 shuffles, residual, packing: latency-bound with eight warps) overlap. 18 warps
// leave 113 registers per thread, so a thread takes its 32 channels in two passes of 16. Per launch at 1024 images,
// without / with residual: 0.199 / 0.238 ms, against 0.201 / 0.258 with one set of eight warps x 32 channels and
// 0.211 / 0.268 with sixteen warps x 16 channels on one accumulator.
constexpr int kThreads = 64 + 2 * 256;  // producer warp, MMA warp, two sets of eight epilogue warps
constexpr int kC = 64;      // input channels = one 128-byte row
constexpr int kO = 64;      // output channels
constexpr int kBN = 3 * kO; // MMA N: the three filter rows side by side
constexpr int kTileW = 8;
constexpr int kRows = 16;             // input rows (= accumulator rows per column) per tile
constexpr int kOutRows = kRows - 2;   // output rows per tile
constexpr int kHaloW = kTileW + 2;
constexpr int kHaloBytes = kHaloW * kRows * 128;  // 20480
constexpr int kTapBytes = kBN * 128;              // weights of one tap column: 24576
constexpr int kWeightBytes = 3 * kTapBytes;       // 73728
constexpr int kStages = 4;
constexpr int kAccStride = 256;                   // TMEM columns between the two accumulators (192 used)
// The epilogue moves whole tiles with TMA: the residual tile comes into a ring of kResBufs boxes, the finished output
// tile leaves from one of kOutBufs boxes; all are [column][row][channel] boxes of 8 x 14 pixels, SWIZZLE_128B.
constexpr int kBoxBytes = kTileW * kOutRows * 128;  // 14336
constexpr int kResBufs = 3;
constexpr int kOutBufs = 2;
constexpr int kSmemBytes = kWeightBytes + kStages * kHaloBytes + (kResBufs + kOutBufs) * kBoxBytes + 1024;
constexpr int kEpiThreads = 256;

__global__ void __launch_bounds__(kThreads, 1) conv3x3_rowstack_kernel(const __grid_constant__ TcParams p) {
    constexpr uint32_t kTmemCols = 2 * kAccStride;
    constexpr uint32_t kIdesc = make_instr_desc(kFmtBF16, kAccF32, kBN);

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_w;
    __shared__ __align__(8) uint64_t bar_full[kStages];
    __shared__ __align__(8) uint64_t bar_empty[kStages];
    __shared__ __align__(8) uint64_t bar_acc_full[2];
    __shared__ __align__(8) uint64_t bar_acc_empty[2];
    __shared__ __align__(8) uint64_t bar_res_full[kResBufs];
    __shared__ __align__(8) uint64_t bar_res_empty[kResBufs];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t w_smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t halo_smem = w_smem + kWeightBytes;
    const uint32_t res_smem = halo_smem + kStages * kHaloBytes;
    const uint32_t out_smem = res_smem + kResBufs * kBoxBytes;
    const bool has_res = p.residual != nullptr;

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
        for (int b = 0; b < kResBufs; ++b) {
            mbar_init(smem_u32(&bar_res_full[b]), 1);
            mbar_init(smem_u32(&bar_res_empty[b]), 8);  // one arrival per warp of the set that read it
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int* abort_ptr = &abort_flag;
    pdl_launch_dependents();

    const int total_tiles = p.tiles_w * p.tiles_h * p.tiles_n;

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&p.tmA[0]);
            tma_prefetch_desc(&p.tmB);
            if (has_res) tma_prefetch_desc(&p.tmA[1]);
            // resident weights: for each tap column kw the rows of filter rows 0, 1, 2 one after the other
            mbar_arrive_expect_tx(smem_u32(&bar_w), kWeightBytes);
            for (int kw = 0; kw < 3; ++kw)
                for (int r = 0; r < 3; ++r)
                    tma_load_2d(w_smem + kw * kTapBytes + r * (kO * 128), &p.tmB, smem_u32(&bar_w), (r * 3 + kw) * kC, 0);
            pdl_wait();  // the weights are constants; the activations come from the previous kernel
            int stage = 0, rb = 0;
            uint32_t phase = 0, rphase = 0;
            for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
                int r = p.reverse ? total_tiles - 1 - tile : tile;
                const int tw = r % p.tiles_w; r /= p.tiles_w;
                const int th = r % p.tiles_h;
                const int tn = r / p.tiles_h;
                if (!mbar_wait_bounded(smem_u32(&bar_empty[stage]), phase ^ 1u, abort_ptr)) break;
                const uint32_t full = smem_u32(&bar_full[stage]);
                mbar_arrive_expect_tx(full, kHaloBytes);
                // tensor map dimensions: channel, ROW, column, image
                tma_load_4d(halo_smem + stage * kHaloBytes, &p.tmA[0], full, 0, th * kOutRows - 1, tw * kTileW - 1, tn);
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
                if (has_res) {  // the residual pixels of the same output tile, two to three tiles ahead of their use
                    if (!mbar_wait_bounded(smem_u32(&bar_res_empty[rb]), rphase ^ 1u, abort_ptr)) break;
                    const uint32_t rfull = smem_u32(&bar_res_full[rb]);
                    mbar_arrive_expect_tx(rfull, kBoxBytes);
                    tma_load_4d(res_smem + rb * kBoxBytes, &p.tmA[1], rfull, 0, th * kOutRows, tw * kTileW, tn);
                    if (++rb == kResBufs) { rb = 0; rphase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = mbar_wait_bounded(smem_u32(&bar_w), 0, abort_ptr);
            const uint32_t hi = desc_hi(1024, kLayoutSw128);  // both operands: 8-row groups of contiguous 128-byte rows
            const uint32_t b_lo0 = desc_lo(w_smem, 16);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                if (!mbar_wait_bounded(smem_u32(&bar_acc_empty[acc]), acc_phase ^ 1u, abort_ptr)) break;
                if (!mbar_wait_bounded(smem_u32(&bar_full[stage]), phase, abort_ptr)) break;
                tc_fence_after_sync();
                const uint32_t d = tmem_base + (uint32_t)(acc * kAccStride);
                const uint32_t a_lo0 = desc_lo(halo_smem + stage * kHaloBytes, 16);
#pragma unroll
                for (int kw = 0; kw < 3; ++kw) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint32_t a_lo = a_lo0 + (uint32_t)((kw * (kRows * 128) + k * 32) >> 4);
                        const uint32_t b_lo = b_lo0 + (uint32_t)((kw * kTapBytes + k * 32) >> 4);
                        umma_f16_split(d, a_lo, hi, b_lo, hi, kIdesc, (kw | k) != 0 ? 1u : 0u);
                    }
                }
                umma_commit(smem_u32(&bar_empty[stage]));
                umma_commit(smem_u32(&bar_acc_full[acc]));
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
    } else {
        const int quad = warp & 3;
        const int half = ((warp - 2) >> 2) & 1;  // output channels [32*half, 32*half+32)
        const int set = (warp - 2) >> 3;
        const int h_l = lane & 15;               // accumulator row = input row of the tile
        const int w_l = 2 * quad + (lane >> 4);
        const bool issuer = threadIdx.x == 64 + set * kEpiThreads;  // owns this set's TMA stores (async groups)
        // this thread's pixel inside an 8 x 14 box ([column][row][channel], 128-byte rows, SWIZZLE_128B: the 16-byte
        // chunk j of a row sits at chunk j ^ (row index & 7); the boxes are 1024-byte aligned)
        const bool in_box = (h_l >= 1) && (h_l <= kOutRows);
        const uint32_t box_row = (uint32_t)(w_l * kOutRows + (h_l - 1));
        const uint32_t row_off = box_row * 128u;
        const uint32_t sw = box_row & 7u;
        const uint32_t out_box = out_smem + set * kBoxBytes;  // kOutBufs == 2: one box per set
        pdl_wait();
        uint32_t acc_phase = 0;
        int it = set;
        for (int tile = blockIdx.x + set * gridDim.x; tile < total_tiles; tile += 2 * gridDim.x, it += 2) {
            int r = p.reverse ? total_tiles - 1 - tile : tile;
            const int tw = r % p.tiles_w; r /= p.tiles_w;
            const int th = r % p.tiles_h;
            const int n = r / p.tiles_h;
            const int rb = it % kResBufs;  // the residual ring is filled in tile order
            const uint32_t rphase = (uint32_t)(it / kResBufs) & 1u;
            // A wait that runs out must not leave some of the set's warps behind at the barriers below: the failure is
            // carried to the first barrier, where all of them learn of it and leave together.
            bool bad = !__all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&bar_acc_full[set]), acc_phase, abort_ptr));
            if (has_res && !bad) bad = !__all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&bar_res_full[rb]), rphase, abort_ptr));
            // this set's output box must have been read by its previous TMA store before it is overwritten
            if (issuer) bulk_wait_group_read<0>();
            if (named_barrier_or(1 + 2 * set, kEpiThreads, bad)) break;
            tc_fence_after_sync();
#pragma unroll
            for (int hp = 0; hp < 2; ++hp) {
                const int c0 = half * 32 + hp * 16;
                const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(set * kAccStride + c0);
                uint32_t v0[16], v1[16], v2[16];
                tmem_ld_32x16(t_addr, v0);           // D_0: wanted by the row below
                tmem_ld_32x16(t_addr + kO, v1);      // D_1: this row
                tmem_ld_32x16(t_addr + 2 * kO, v2);  // D_2: wanted by the row above
                tmem_ld_wait();
                if (hp == 1) {  // accumulator is in registers now
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[set]));
                }
                float f[16];
#pragma unroll
                for (int j = 0; j < 16; j += 4) {
                    const float4 b = p.bias != nullptr ? __ldg(reinterpret_cast<const float4*>(p.bias + c0 + j)) : make_float4(0.f, 0.f, 0.f, 0.f);
                    const float bb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float up = __uint_as_float(__shfl_up_sync(0xffffffffu, v0[j + k], 1));      // D_0 of row oh - 1
                        const float down = __uint_as_float(__shfl_down_sync(0xffffffffu, v2[j + k], 1));  // D_2 of row oh + 1
                        f[j + k] = __fadd_rn(__fadd_rn(__fadd_rn(up, __uint_as_float(v1[j + k])), down), bb[k]);
                    }
                }
                if (has_res && in_box) {
                    const uint32_t base = res_smem + rb * kBoxBytes + row_off;
#pragma unroll
                    for (int g = 0; g < 2; ++g) {
                        const uint4 rv = ld_shared_v4(base + ((((uint32_t)(half * 4 + hp * 2 + g)) ^ sw) << 4));
                        const uint32_t w[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            f[g * 8 + 2 * k] = __fadd_rn(f[g * 8 + 2 * k], bf16_lo(w[k]));
                            f[g * 8 + 2 * k + 1] = __fadd_rn(f[g * 8 + 2 * k + 1], bf16_hi(w[k]));
                        }
                    }
                }
                if (p.relu) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) f[j] = f[j] > 0.0f ? f[j] : 0.0f;
                }
                if (in_box) {
                    const uint32_t base = out_box + row_off;
#pragma unroll
                    for (int g = 0; g < 2; ++g) {
                        uint4 o;
                        o.x = pack_bf16(f[g * 8 + 0], f[g * 8 + 1]);
                        o.y = pack_bf16(f[g * 8 + 2], f[g * 8 + 3]);
                        o.z = pack_bf16(f[g * 8 + 4], f[g * 8 + 5]);
                        o.w = pack_bf16(f[g * 8 + 6], f[g * 8 + 7]);
                        st_shared_v4(base + ((((uint32_t)(half * 4 + hp * 2 + g)) ^ sw) << 4), o);
                    }
                }
            }
            if (has_res) {
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bar_res_empty[rb]));
            }
            fence_proxy_async_shared();
            named_barrier(2 + 2 * set, kEpiThreads);
            if (issuer) {  // pixels beyond the image's last row or column are clipped by the store
                tma_store_4d(&p.tmA[2], out_box, 0, th * kOutRows, tw * kTileW, n);
                bulk_commit_group();
            }
            acc_phase ^= 1u;
        }
        if (issuer) bulk_wait_group_all();
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
// int8 form (tcgen05 kind::i8, int32 accumulators, fixed-point requantize): the same tiling with 64-byte pixels.
// The general implicit-GEMM kernel fetches every input pixel nine times in boxes of 64-byte rows, and at 64 bytes per
// row the copy engine's row rate, not bandwidth, bounds it (~4 cycles per row measured: 170 us for 256 images of
// 56 x 56). Here a tile is ONE box of 160 rows; six instructions of N = 192, K = 32 bytes do its 3 x 3 x 64 reduction.
// The sum over the three filter rows is an int32 sum (exact in any order), the result is requantized and stored by the
// thread that owns the pixel (32 bytes per thread, no staging).
constexpr int kPx8 = 64;                                // bytes per int8 pixel
constexpr int kHaloBytes8 = kHaloW * kRows * kPx8;      // 10240
constexpr int kTapBytes8 = kBN * kPx8;                  // 12288
constexpr int kWeightBytes8 = 3 * kTapBytes8;           // 36864
constexpr int kStages8 = 6;
constexpr int kSmemBytes8 = kWeightBytes8 + kStages8 * kHaloBytes8 + 1024;
// Two sets of eight epilogue warps, one per accumulator: the epilogue (three TMEM loads, 64 shuffles and the requantize
// per thread) is latency-bound with eight warps (2900 cycles per tile against ~900 issue cycles), so consecutive tiles
// are drained concurrently. 18 warps leave 113 registers per thread: a thread takes its 32 channels in two passes of 16.
constexpr int kThreads8 = 64 + 2 * 256;

__global__ void __launch_bounds__(kThreads8, 1) conv3x3_rowstack_s8_kernel(const __grid_constant__ TcParams p) {
    constexpr uint32_t kTmemCols = 2 * kAccStride;
    constexpr uint32_t kIdesc = make_instr_desc(kFmtS8, kAccS32, kBN);

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_w;
    __shared__ __align__(8) uint64_t bar_full[kStages8];
    __shared__ __align__(8) uint64_t bar_empty[kStages8];
    __shared__ __align__(8) uint64_t bar_acc_full[2];
    __shared__ __align__(8) uint64_t bar_acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    // per output channel the constants of the high-word requantize (requant_prepare), prepared once; q_fast = 0 when
    // some channel does not qualify (the general formula is used then)
    __shared__ __align__(16) int4 q_tab[kO];
    __shared__ int q_fast;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t w_smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t halo_smem = w_smem + kWeightBytes8;

    if (threadIdx.x == 0) q_fast = 1;
    __syncthreads();
    if (threadIdx.x >= 64 && threadIdx.x < 64 + kO) {  // the quantization constants are call arguments, not a producer's output
        const int c = threadIdx.x - 64;
        // |accumulator| <= 128 * 128 * (9 taps * 64 channels)
        if (!requant_prepare(__ldg(p.bias_i32 + c), __ldg(p.multiplier + c), __ldg(p.shift + c), 128ll * 128 * 9 * kC, &q_tab[c])) q_fast = 0;
    }
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar_w), 1);
        for (int s = 0; s < kStages8; ++s) {
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
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int* abort_ptr = &abort_flag;
    pdl_launch_dependents();

    const int total_tiles = p.tiles_w * p.tiles_h * p.tiles_n;

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&p.tmA[0]);
            tma_prefetch_desc(&p.tmB);
            mbar_arrive_expect_tx(smem_u32(&bar_w), kWeightBytes8);
            for (int kw = 0; kw < 3; ++kw)
                for (int r = 0; r < 3; ++r)
                    tma_load_2d(w_smem + kw * kTapBytes8 + r * (kO * kPx8), &p.tmB, smem_u32(&bar_w), (r * 3 + kw) * kC, 0);
            pdl_wait();
            int stage = 0;
            uint32_t phase = 0;
            for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
                int r = tile;
                const int tw = r % p.tiles_w; r /= p.tiles_w;
                const int th = r % p.tiles_h;
                const int tn = r / p.tiles_h;
                if (!mbar_wait_bounded(smem_u32(&bar_empty[stage]), phase ^ 1u, abort_ptr)) break;
                const uint32_t full = smem_u32(&bar_full[stage]);
                mbar_arrive_expect_tx(full, kHaloBytes8);
                tma_load_4d(halo_smem + stage * kHaloBytes8, &p.tmA[0], full, 0, th * kOutRows - 1, tw * kTileW - 1, tn);
                if (++stage == kStages8) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = mbar_wait_bounded(smem_u32(&bar_w), 0, abort_ptr);
            const uint32_t hi = desc_hi(8 * kPx8, kLayoutSw64);  // both operands: 8-row groups of contiguous 64-byte rows
            const uint32_t b_lo0 = desc_lo(w_smem, 16);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                if (!mbar_wait_bounded(smem_u32(&bar_acc_empty[acc]), acc_phase ^ 1u, abort_ptr)) break;
                if (!mbar_wait_bounded(smem_u32(&bar_full[stage]), phase, abort_ptr)) break;
                tc_fence_after_sync();
                const uint32_t d = tmem_base + (uint32_t)(acc * kAccStride);
                const uint32_t a_lo0 = desc_lo(halo_smem + stage * kHaloBytes8, 16);
#pragma unroll
                for (int kw = 0; kw < 3; ++kw) {
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const uint32_t a_lo = a_lo0 + (uint32_t)((kw * (kRows * kPx8) + k * 32) >> 4);
                        const uint32_t b_lo = b_lo0 + (uint32_t)((kw * kTapBytes8 + k * 32) >> 4);
                        umma_i8_split(d, a_lo, hi, b_lo, hi, kIdesc, (kw | k) != 0 ? 1u : 0u);
                    }
                }
                umma_commit(smem_u32(&bar_empty[stage]));
                umma_commit(smem_u32(&bar_acc_full[acc]));
                if (++stage == kStages8) { stage = 0; phase ^= 1u; }
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
    } else {
        const int quad = warp & 3;
        const int half = ((warp - 2) >> 2) & 1;  // output channels [32*half, 32*half+32)
        const int set = (warp - 2) >> 3;         // the accumulator this warp drains: tiles of that parity
        const int h_l = lane & 15;               // accumulator row = input row of the tile
        const int w_l = 2 * quad + (lane >> 4);
        const bool in_box = (h_l >= 1) && (h_l <= kOutRows);
        int8_t* out = static_cast<int8_t*>(p.out);
        const int32_t lo = p.relu ? 0 : INT32_MIN;
        const bool fast = q_fast != 0;
        pdl_wait();
        uint32_t acc_phase = 0;
        // this set's tiles: blockIdx.x + (2 i + set) gridDim.x; the tile coordinates advance by a fixed step with carries
        const int step = 2 * (int)gridDim.x;
        const int s_tw = step % p.tiles_w, s_th = (step / p.tiles_w) % p.tiles_h, s_n = step / (p.tiles_w * p.tiles_h);
        int tile = (int)blockIdx.x + set * (int)gridDim.x;
        int tw = tile % p.tiles_w, th = (tile / p.tiles_w) % p.tiles_h, n = tile / (p.tiles_w * p.tiles_h);
        for (; tile < total_tiles; tile += step) {
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&bar_acc_full[set]), acc_phase, abort_ptr))) break;
            tc_fence_after_sync();
            const int oh = th * kOutRows + h_l - 1, ow = tw * kTileW + w_l;
            const bool store = in_box && oh < p.OH && ow < p.OW;
            int8_t* dst = out + (((size_t)n * p.OH + oh) * p.OW + ow) * kO;
#pragma unroll
            for (int hp = 0; hp < 2; ++hp) {
                const int c0 = half * 32 + hp * 16;
                const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(set * kAccStride + c0);
                uint32_t v0[16], v1[16], v2[16];
                tmem_ld_32x16(t_addr, v0);           // D_0: wanted by the row below
                tmem_ld_32x16(t_addr + kO, v1);      // D_1: this row
                tmem_ld_32x16(t_addr + 2 * kO, v2);  // D_2: wanted by the row above
                tmem_ld_wait();
                if (hp == 1) {  // the accumulator is in registers now
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[set]));
                }
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    v1[j] += __shfl_up_sync(0xffffffffu, v0[j], 1) + __shfl_down_sync(0xffffffffu, v2[j], 1);
                uint32_t qw[4];
                if (fast) {
#pragma unroll
                    for (int j = 0; j < 16; j += 4) {
                        const uint32_t vv[4] = {v1[j], v1[j + 1], v1[j + 2], v1[j + 3]};
                        // (the same addresses in every lane: broadcasts)
                        const int4 qq[4] = {q_tab[c0 + j], q_tab[c0 + j + 1], q_tab[c0 + j + 2], q_tab[c0 + j + 3]};
                        qw[j >> 2] = requant4_prepared(vv, qq, lo);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) qw[j] = 0;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int8_t x = requantize_s8((int32_t)(v1[j] + (uint32_t)__ldg(p.bias_i32 + c0 + j)), __ldg(p.multiplier + c0 + j),
                                                       __ldg(p.shift + c0 + j), p.relu);
                        qw[j >> 2] |= (uint32_t)(uint8_t)x << (8 * (j & 3));
                    }
                }
                if (store) *reinterpret_cast<uint4*>(dst + c0) = make_uint4(qw[0], qw[1], qw[2], qw[3]);
            }
            acc_phase ^= 1u;
            tw += s_tw;
            if (tw >= p.tiles_w) { tw -= p.tiles_w; ++th; }
            th += s_th;
            if (th >= p.tiles_h) { th -= p.tiles_h; ++n; }
            n += s_n;
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

}  // namespace

bool rowstack3x3_applicable(TcDType dtype, int C, int O, int KH, int KW, int stride, int pad_h, int pad_w, int dil_h, int dil_w,
                            int H, int W) {
    // the row-first tensor map needs both pixel strides to be multiples of 16 bytes (always true: 128-byte pixels)
    return dtype == kTcBF16 && C == kC && O == kO && KH == 3 && KW == 3 && stride == 1 && pad_h == 1 && pad_w == 1 &&
           dil_h == 1 && dil_w == 1 && H >= 1 && W >= 1;
}

int32_t rowstack3x3_setup(TcParams* p, const void* act_nhwc, const void* w_packed, int N, int H, int W) {
    p->N = N; p->OH = H; p->OW = W; p->Cout = kO;
    p->taps_h = 3; p->taps_w = 3; p->stride = 1; p->pad_h = 1; p->pad_w = 1; p->dil_h = 1; p->dil_w = 1;
    p->cblocks = 1; p->kb_elems = kC;
    p->BW = kTileW; p->BH = kOutRows; p->BNI = 1;
    p->tiles_w = (W + kTileW - 1) / kTileW;
    p->tiles_h = (H + kOutRows - 1) / kOutRows;
    p->tiles_n = N;
    p->tiles_c = 1;
    const uint64_t px = kC * 2;
    // dimensions: channel, ROW, column, image -> the box lands in shared memory as [column][row][channel]
    const uint64_t dims[4] = {(uint64_t)kC, (uint64_t)H, (uint64_t)W, (uint64_t)N};
    const uint64_t strides[3] = {(uint64_t)W * px, px, (uint64_t)H * W * px};
    const uint32_t box[4] = {(uint32_t)kC, (uint32_t)kRows, (uint32_t)kHaloW, 1u};
    KXC_TRY(tc_make_tmap(&p->tmA[0], kTcBF16, 4, const_cast<void*>(act_nhwc), dims, strides, box, 128));
    for (int i = 1; i < 4; ++i) p->tmA[i] = p->tmA[0];
    const uint64_t ktot = (uint64_t)9 * kC;
    const uint64_t bdims[2] = {ktot, (uint64_t)kO};
    const uint64_t bstr[1] = {ktot * 2};
    const uint32_t bbox[2] = {(uint32_t)kC, (uint32_t)kO};
    KXC_TRY(tc_make_tmap(&p->tmB, kTcBF16, 2, const_cast<void*>(w_packed), bdims, bstr, bbox, 128));
    KXC_TRY(tc_status_word(&p->status));
    return KXC_B200_OK;
}

bool rowstack3x3_s8_applicable(int C, int O, int KH, int KW, int stride, int pad_h, int pad_w, int dil_h, int dil_w) {
    return C == kC && O == kO && KH == 3 && KW == 3 && stride == 1 && pad_h == 1 && pad_w == 1 && dil_h == 1 && dil_w == 1;
}

int32_t rowstack3x3_s8_setup(TcParams* p, const void* act_nhwc, const void* w_packed, int N, int H, int W) {
    p->N = N; p->OH = H; p->OW = W; p->Cout = kO;
    p->taps_h = 3; p->taps_w = 3; p->stride = 1; p->pad_h = 1; p->pad_w = 1; p->dil_h = 1; p->dil_w = 1;
    p->cblocks = 1; p->kb_elems = kC;
    p->BW = kTileW; p->BH = kOutRows; p->BNI = 1;
    p->tiles_w = (W + kTileW - 1) / kTileW;
    p->tiles_h = (H + kOutRows - 1) / kOutRows;
    p->tiles_n = N;
    p->tiles_c = 1;
    const uint64_t px = kPx8;
    const uint64_t dims[4] = {(uint64_t)kC, (uint64_t)H, (uint64_t)W, (uint64_t)N};
    const uint64_t strides[3] = {(uint64_t)W * px, px, (uint64_t)H * W * px};
    const uint32_t box[4] = {(uint32_t)kC, (uint32_t)kRows, (uint32_t)kHaloW, 1u};
    KXC_TRY(tc_make_tmap(&p->tmA[0], kTcS8, 4, const_cast<void*>(act_nhwc), dims, strides, box, kPx8));
    for (int i = 1; i < 4; ++i) p->tmA[i] = p->tmA[0];
    const uint64_t ktot = (uint64_t)9 * kC;
    const uint64_t bdims[2] = {ktot, (uint64_t)kO};
    const uint64_t bstr[1] = {ktot};
    const uint32_t bbox[2] = {(uint32_t)kC, (uint32_t)kO};
    KXC_TRY(tc_make_tmap(&p->tmB, kTcS8, 2, const_cast<void*>(w_packed), bdims, bstr, bbox, kPx8));
    KXC_TRY(tc_status_word(&p->status));
    return KXC_B200_OK;
}

int32_t rowstack3x3_s8_launch(const TcParams& p, cudaStream_t stream) {
    static PerDeviceOnce smem_once;
    KXC_TRY(smem_opt_in(smem_once, conv3x3_rowstack_s8_kernel, kSmemBytes8));
    if (!p.vec_ok || p.out == nullptr) return fail(KXC_B200_ERR_INVALID, "row-stacked 3x3 int8 conv: pointers must be 16-byte aligned");
    const long long tiles = (long long)p.tiles_w * p.tiles_h * p.tiles_n;
    if (tiles <= 0) return KXC_B200_OK;
    const int grid = (int)(tiles < kNumSMs ? tiles : kNumSMs);
    KXC_CUDA_TRY(launch_kernel(conv3x3_rowstack_s8_kernel, dim3(grid), dim3(kThreads8), kSmemBytes8, stream, /*pdl=*/true, 1, p));
    return check_launch("conv3x3_rowstack_s8_kernel");
}

int32_t rowstack3x3_bind(TcParams* p) {
    // tmA[1]: residual tiles (loads), tmA[2]: output tiles (stores); same tensor geometry as the input, 8 x 14 boxes
    if (p->out == nullptr) return fail(KXC_B200_ERR_INVALID, "row-stacked 3x3 conv: no output tensor");
    const uint64_t px = kC * 2;
    const uint64_t dims[4] = {(uint64_t)kO, (uint64_t)p->OH, (uint64_t)p->OW, (uint64_t)p->N};
    const uint64_t strides[3] = {(uint64_t)p->OW * px, px, (uint64_t)p->OH * p->OW * px};
    const uint32_t box[4] = {(uint32_t)kO, (uint32_t)kOutRows, (uint32_t)kTileW, 1u};
    KXC_TRY(tc_make_tmap(&p->tmA[2], kTcBF16, 4, p->out, dims, strides, box, 128));
    if (p->residual != nullptr)
        KXC_TRY(tc_make_tmap(&p->tmA[1], kTcBF16, 4, const_cast<void*>(p->residual), dims, strides, box, 128));
    return KXC_B200_OK;
}

int32_t rowstack3x3_launch(const TcParams& p, cudaStream_t stream) {
    static PerDeviceOnce smem_once;
    KXC_TRY(smem_opt_in(smem_once, conv3x3_rowstack_kernel, kSmemBytes));
    if (!p.vec_ok || p.out == nullptr) return fail(KXC_B200_ERR_INVALID, "row-stacked 3x3 conv: pointers must be 16-byte aligned");
    const long long tiles = (long long)p.tiles_w * p.tiles_h * p.tiles_n;
    if (tiles <= 0) return KXC_B200_OK;
    const int grid = (int)(tiles < kNumSMs ? tiles : kNumSMs);
    KXC_CUDA_TRY(launch_kernel(conv3x3_rowstack_kernel, dim3(grid), dim3(kThreads), kSmemBytes, stream, /*pdl=*/true, 1, p));
    return check_launch("conv3x3_rowstack_kernel");
}

}  // namespace kxc_b200

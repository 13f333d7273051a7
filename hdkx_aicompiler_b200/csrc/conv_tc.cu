// Implicit-GEMM convolution / dense on tcgen05 tensor cores with TMEM accumulators and TMA operand
// loads (see conv_tc.cuh for the GEMM view). Persistent, warp-specialised CTAs, one per SM:
//
//   warp 0      TMA producer   one lane issues cp.async.bulk.tensor loads into a ring of swizzled
//                              shared-memory stages, each guarded by a full/empty mbarrier pair
//   warp 1      MMA issuer     one lane issues tcgen05.mma (M = 128, N = BN, K = 32 bytes per
//                              instruction) into one of two TMEM accumulators; tcgen05.commit
//                              releases stages and publishes finished accumulators; owns TMEM alloc
//   warps 2..9  epilogue       tcgen05.ld the accumulator (two warps per 32-lane quadrant, each half
//                              of the columns),
//                              +bias -> +residual -> ReLU (or int8 requantize), store; overlaps the
//                              next tile's main loop through the second accumulator
//
// Every wait is bounded (sm100::mbar_wait_bounded); a wait that runs out sets the CTA's abort flag
// and the global status word, every role leaves its loop, TMEM is released and the kernel returns.
#include "conv_tc.cuh"

#include <cuda_bf16.h>
#include <cudaTypedefs.h>

#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "conv_epilogue.cuh"
#include "sm100.cuh"

namespace kxc_b200 {
namespace {

using namespace sm100;

constexpr int kTcThreads = 320;  // 2 control warps + 8 epilogue warps
constexpr int kStoreBoxBytes = 32 * 128;
constexpr int kSmemLimit = 227 * 1024;

template <int KB_BYTES, int BN, int kCtas, int kMT = 1>
struct StageGeom {
    static constexpr int kATileBytes = 128 * KB_BYTES;
    static constexpr int kABytes = kMT * kATileBytes;  // kMT pixel tiles share one B tile
    static constexpr int kBBytes = (BN / kCtas) * KB_BYTES;  // a CTA of a pair holds half of the B tile's rows
    static constexpr int kStageBytes = kABytes + kBBytes;
    // per epilogue warp a 4 KiB box (32 pixels x 64 channels, SWIZZLE_128B) that TMA stores read; its first half
    // doubles as the staging tile of the per-thread store path
    static constexpr int kEpilogueBytes = 8 * kStoreBoxBytes;
    static constexpr int kStagesRaw = (kSmemLimit - 2048 - kEpilogueBytes) / kStageBytes;
    static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
    static constexpr int kSmemBytes = kStages * kStageBytes + kEpilogueBytes + 1024;  // + slack to align the ring to 1024 B
};

// kCtas = 2: the CTAs of a cluster of two work as a pair on 256 output pixels x BN channels. Each loads its own
// 128-pixel A tile and HALF of the B tile; the leader (cluster rank 0) issues tcgen05.mma.cta_group::2
// (M = 256), which reads both CTAs' shared memory and writes each CTA's 128 rows into that CTA's TMEM.
// Both CTAs' loads count on the leader's "full" barrier; commits arrive on both CTAs' barriers; the
// peer's epilogue warps release accumulators on the leader's "accumulator empty" barrier.
//
// kDual: a second output, the 1x1 convolution of the same stride over the same input (TcParams::tmB2 ...). Its
// reduction is appended to the K loop as `cblocks` extra stages that load the centre tap's pixels again together
// with the second weight tensor's rows and accumulate into a second TMEM accumulator; the epilogue drains both.
//
// kMT = 2: a work item is TWO pixel tiles per CTA against one B tile. Their MMAs alternate between two
// accumulators, which gives the tensor core two independent accumulate chains (a pair's M = 256 instruction has
// a long dependent-issue latency) and halves the B traffic per pixel.
template <MmaKind kKind, int KB_BYTES, int BN, int kOutMode, int kCtas, bool kDual = false, int kMT = 1>
__global__ void __launch_bounds__(kTcThreads, 1) conv_igemm_kernel(const __grid_constant__ TcParams p) {
    using G = StageGeom<KB_BYTES, BN, kCtas, kMT>;
    static_assert(!(kDual && kMT != 1), "the two-output kernel works on one pixel tile at a time");
    constexpr bool kPair = kCtas == 2;
    constexpr int kStages = G::kStages;
    constexpr int kAccCols = (kDual ? 2 : kMT) * BN;  // TMEM columns of one accumulator buffer
    // two accumulator buffers (the epilogue of one work item overlaps the next item's main loop) where TMEM's 512
    // columns allow it, else one
    constexpr int kBufs = 2 * kAccCols <= 512 ? 2 : 1;
    constexpr uint32_t kTmemUsed = kBufs * kAccCols;
    constexpr uint32_t kTmemCols = kTmemUsed <= 128 ? 128u : (kTmemUsed <= 256 ? 256u : 512u);  // allocations are powers of two
    static_assert(kTmemUsed <= 512, "TMEM has 512 columns");
    static_assert(!kDual || (!kPair && kOutMode == kOutNHWC_BF16), "the dual kernel exists for single CTAs and bf16 NHWC output");
    constexpr uint32_t kIdesc =
        make_instr_desc(kKind == MmaKind::F16 ? kFmtBF16 : (kKind == MmaKind::TF32 ? kFmtTF32 : kFmtS8),
                        kKind == MmaKind::I8 ? kAccS32 : kAccF32, BN, 128u * kCtas);

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[kStages];
    __shared__ __align__(8) uint64_t bar_empty[kStages];
    __shared__ __align__(8) uint64_t bar_acc_full[2];
    __shared__ __align__(8) uint64_t bar_acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t cta_rank = kPair ? cluster_cta_rank() : 0u;
    const bool leader = cta_rank == 0;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bar_acc_full[a]), 1);
            mbar_init(smem_u32(&bar_acc_empty[a]), 8 * kCtas);  // one arrival per epilogue warp (of both CTAs)
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        if constexpr (kPair) {
            tmem_alloc_pair(smem_u32(&tmem_base_slot), kTmemCols);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
            tmem_relinquish();
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if constexpr (kPair) cluster_sync_all();  // the peer's barriers are initialised before anything signals them
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int* abort_ptr = &abort_flag;
    pdl_launch_dependents();  // the next kernel's CTAs may take over SMs this grid has left; they wait before touching memory

    const int num_kb_main = p.taps_h * p.taps_w * p.cblocks;
    const int num_kb = num_kb_main + (kDual ? p.cblocks : 0);
    // Work items: (channel tile, group of kCtas consecutive pixel tiles). A pair whose second pixel tile
    // does not exist loads a box beyond the last image (all zeros) and stores nothing for it.
    const int m_tiles = p.tiles_w * p.tiles_h * p.tiles_n;
    const int total_tiles = p.tiles_c * ((m_tiles + kCtas * kMT - 1) / (kCtas * kMT));
    const int first_tile = kPair ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int tile_step = kPair ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    const int rows_used = p.BW * p.BH * p.BNI;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&p.tmB);
            tma_prefetch_desc(&p.tmA[0]);
            if constexpr (kDual) tma_prefetch_desc(&p.tmB2);
            const uint32_t tx_bytes = (uint32_t)(kMT * rows_used * KB_BYTES + G::kBBytes);
            pdl_wait();  // the activations come from the previous kernel
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int item = first_tile; ok && item < total_tiles; item += tile_step) {
                const int tile = p.reverse ? total_tiles - 1 - item : item;
                const int ct = tile % p.tiles_c;
                int ow0[kMT], oh0[kMT], n0[kMT];
#pragma unroll
                for (int t = 0; t < kMT; ++t) {
                    int r = ((tile / p.tiles_c) * kCtas + (int)cta_rank) * kMT + t;
                    const int tw = r % p.tiles_w; r /= p.tiles_w;
                    const int th = r % p.tiles_h;
                    const int tn = r / p.tiles_h;
                    ow0[t] = tw * p.BW; oh0[t] = th * p.BH; n0[t] = tn * p.BNI;
                }
                const int co0 = ct * BN + (int)cta_rank * (BN / kCtas);
                int kb = 0;
                for (int kh = 0; ok && kh < p.taps_h; ++kh) {
                    for (int kw = 0; ok && kw < p.taps_w; ++kw) {
                        const int dh = kh * p.dil_h - p.pad_h;
                        const int dw = kw * p.dil_w - p.pad_w;
                        int map = 0, ch = dh, cw = dw;  // offsets of this tap's box from the tile's first pixel
                        if (p.stride == 2) {
                            const int hp = dh & 1, wp = dw & 1;
                            map = hp * 2 + wp;
                            ch = (dh - hp) >> 1;
                            cw = (dw - wp) >> 1;
                        }
                        for (int cb = 0; cb < p.cblocks; ++cb, ++kb) {
                            if (!mbar_wait_bounded(smem_u32(&bar_empty[stage]), phase ^ 1u, abort_ptr)) {
                                ok = false;
                                break;
                            }
                            const uint32_t full = smem_u32(&bar_full[stage]);
                            const uint32_t a_dst = ring + (uint32_t)stage * G::kStageBytes;
                            if constexpr (kPair) {
                                if (leader) mbar_arrive_expect_tx(full, 2u * tx_bytes);
                                const uint32_t full0 = map_to_cta(full, 0);
#pragma unroll
                                for (int t = 0; t < kMT; ++t)
                                    tma_load_4d_pair(a_dst + t * G::kATileBytes, &p.tmA[map], full0, cb * p.kb_elems, ow0[t] + cw,
                                                     oh0[t] + ch, n0[t]);
                                tma_load_2d_pair(a_dst + G::kABytes, &p.tmB, full0, kb * p.kb_elems, co0);
                            } else {
                                mbar_arrive_expect_tx(full, tx_bytes);
#pragma unroll
                                for (int t = 0; t < kMT; ++t)
                                    tma_load_4d(a_dst + t * G::kATileBytes, &p.tmA[map], full, cb * p.kb_elems, ow0[t] + cw, oh0[t] + ch,
                                                n0[t]);
                                tma_load_2d(a_dst + G::kABytes, &p.tmB, full, kb * p.kb_elems, co0);
                            }
                            if (++stage == kStages) { stage = 0; phase ^= 1u; }
                        }
                    }
                }
                if constexpr (kDual) {
                    // second output: the centre tap's pixels (the 1x1 convolution's only tap) against tmB2
                    const int dh = (p.taps_h / 2) * p.dil_h - p.pad_h, dw = (p.taps_w / 2) * p.dil_w - p.pad_w;  // 0, 0
                    int map = 0, ch = oh0[0] + dh, cw = ow0[0] + dw;
                    if (p.stride == 2) {
                        const int hp = dh & 1, wp = dw & 1;
                        map = hp * 2 + wp;
                        ch = oh0[0] + ((dh - hp) >> 1);
                        cw = ow0[0] + ((dw - wp) >> 1);
                    }
                    for (int cb = 0; ok && cb < p.cblocks; ++cb) {
                        if (!mbar_wait_bounded(smem_u32(&bar_empty[stage]), phase ^ 1u, abort_ptr)) {
                            ok = false;
                            break;
                        }
                        const uint32_t full = smem_u32(&bar_full[stage]);
                        const uint32_t a_dst = ring + (uint32_t)stage * G::kStageBytes;
                        mbar_arrive_expect_tx(full, tx_bytes);
                        tma_load_4d(a_dst, &p.tmA[map], full, cb * p.kb_elems, cw, ch, n0[0]);
                        tma_load_2d(a_dst + G::kABytes, &p.tmB2, full, cb * p.kb_elems, co0);
                        if (++stage == kStages) { stage = 0; phase ^= 1u; }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0 && leader) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int tile = first_tile; ok && tile < total_tiles; tile += tile_step) {
                if (!mbar_wait_bounded(smem_u32(&bar_acc_empty[acc]), acc_phase ^ 1u, abort_ptr)) break;
                tc_fence_after_sync();
                const uint32_t d_main = tmem_base + (uint32_t)(acc * kAccCols);
                for (int kb = 0; kb < num_kb; ++kb) {
                    const bool second = kDual && kb >= num_kb_main;
                    const uint32_t d_tmem = second ? d_main + (uint32_t)BN : d_main;
                    const int kb_local = second ? kb - num_kb_main : kb;
                    if (!mbar_wait_bounded(smem_u32(&bar_full[stage]), phase, abort_ptr)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t a_addr = ring + (uint32_t)stage * G::kStageBytes;
                    const uint64_t a_desc = make_smem_desc(a_addr, KB_BYTES);
                    const uint64_t b_desc = make_smem_desc(a_addr + G::kABytes, KB_BYTES);
#pragma unroll
                    for (int k = 0; k < KB_BYTES / 32; ++k) {
#pragma unroll
                        for (int t = 0; t < kMT; ++t) {
                            // advancing 32 bytes along K inside the swizzle span = +2 in the (addr >> 4) field;
                            // the next pixel tile of the stage is kATileBytes further on
                            const uint64_t a_k = a_desc + (uint64_t)(2 * k) + (uint64_t)(t * (G::kATileBytes >> 4));
                            const uint32_t d_t = d_tmem + (uint32_t)(t * BN);
                            if constexpr (kPair)
                                umma_pair<kKind>(d_t, a_k, b_desc + (uint64_t)(2 * k), kIdesc, (kb_local | k) != 0 ? 1u : 0u);
                            else
                                umma<kKind>(d_t, a_k, b_desc + (uint64_t)(2 * k), kIdesc, (kb_local | k) != 0 ? 1u : 0u);
                        }
                    }
                    if constexpr (kPair) umma_commit_pair(smem_u32(&bar_empty[stage]), 3);
                    else umma_commit(smem_u32(&bar_empty[stage]));
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                if constexpr (kPair) umma_commit_pair(smem_u32(&bar_acc_full[acc]), 3);
                else umma_commit(smem_u32(&bar_acc_full[acc]));
                if (++acc == kBufs) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
    } else {
        // ------------------------------ epilogue ------------------------------
        const int quad = warp & 3;  // TMEM lanes [32*quad, 32*quad+32) are the ones this warp may read
        const int half = (warp - 2) >> 2;  // which half of the tile's columns this warp handles
        constexpr int kChunksPerWarp = BN / 64;
        const int row = quad * 32 + lane;
        const int box_hw = p.BH * p.BW;
        const int n_l = row / box_hw;
        const int rem = row - n_l * box_hw;
        const int h_l = rem / p.BW;
        const int w_l = rem - h_l * p.BW;
        const bool fast = (kOutMode == kOutNHWC_BF16) && p.vec_ok && ((p.Cout & 31) == 0);
        const bool has_res = p.residual != nullptr;
        const EpiParams ep = {p.bias, p.residual, p.out, p.Cout, p.relu};
        const uint32_t stage_tile = ring + (uint32_t)(kStages * G::kStageBytes) + (uint32_t)((warp - 2) * kStoreBoxBytes);
        // Residual-free launches with store maps: the warp's values go into its swizzled box and leave by TMA store
        // (boxes are 64 channels wide: a warp needs an even number of 32-column chunks, which the 192-wide tile lacks)
        const bool boxed = fast && p.store_box && !has_res && (BN >= 128) && (kChunksPerWarp % 2 == 0);
        pdl_wait();  // residual reads and output writes must not overtake earlier kernels
        int acc = 0;
        uint32_t acc_phase = 0;
        bool alive = true;
        for (int item = first_tile; alive && item < total_tiles; item += tile_step) {
          const int tile = p.reverse ? total_tiles - 1 - item : item;
          const int ct = tile % p.tiles_c;
#pragma unroll 1
          for (int t = 0; t < kMT; ++t) {
            int r = ((tile / p.tiles_c) * kCtas + (int)cta_rank) * kMT + t;
            const int tw = r % p.tiles_w; r /= p.tiles_w;
            const int th = r % p.tiles_h;
            const int tn = r / p.tiles_h;
            const int n = tn * p.BNI + n_l, oh = th * p.BH + h_l, ow = tw * p.BW + w_l;
            const bool valid = (row < rows_used) && (n < p.N) && (oh < p.OH) && (ow < p.OW);
            const size_t pix = ((size_t)n * p.OH + oh) * p.OW + ow;
            const int col0 = half * kChunksPerWarp * 32;  // first column of this warp inside the tile
            const int c_base = ct * BN + col0;
            uint4 res_cur[4] = {};
            RowMap rows;
            if (fast && !boxed) {
                rows = make_row_map(pix, valid, lane);
                if (has_res && c_base < p.Cout) residual_fetch_rows(ep, rows, c_base, lane, res_cur);
            }
            if (t == 0) {
                bool ok = mbar_wait_bounded(smem_u32(&bar_acc_full[acc]), acc_phase, abort_ptr);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    alive = false;
                    break;
                }
                tc_fence_after_sync();
            }
            const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * kAccCols + t * BN + col0);
#pragma unroll 1
            for (int i = 0; i < kChunksPerWarp; ++i) {
                const int c0 = c_base + i * 32;
                uint32_t v[32];
                tmem_ld_32x32(t_addr + (uint32_t)(i * 32), v);
                uint4 res_next[4] = {};
                if (fast && has_res && (i + 1 < kChunksPerWarp) && (c0 + 32 < p.Cout))
                    residual_fetch_rows(ep, rows, c0 + 32, lane, res_next);
                tmem_ld_wait();
                if (boxed) {
                    if ((i & 1) == 0) {  // a new 64-channel group: the previous store must have read the box
                        if (lane == 0) bulk_wait_group_read<0>();
                        __syncwarp();
                    }
                    if (c0 < p.Cout) epilogue_box_bf16(ep, v, c0, stage_tile, (i & 1) * 4, lane);
                    if (i & 1) {
                        fence_proxy_async_shared();
                        __syncwarp();
                        // lane 0's pixel is the first of the warp's 32: the box origin (a pair's missing second tile
                        // lies beyond the last image and stores nothing)
                        if (lane == 0 && c0 < p.Cout && n < p.N) {
                            tma_store_4d(&p.tmOut, stage_tile, c0 - 32, ow, oh, n);
                            bulk_commit_group();
                        }
                    }
                } else if (fast) {
                    if (c0 < p.Cout) epilogue_coalesced_bf16<32>(ep, v, c0, stage_tile, lane, rows, res_cur, has_res);
                } else {
                    epilogue_chunk<kOutMode>(p, v, c0, valid, n, oh, ow);
                }
#pragma unroll
                for (int g = 0; g < 4; ++g) res_cur[g] = res_next[g];
            }
            if constexpr (kDual) {
                // second output: same rows and channels from the accumulator next to the main one; no residual
                const EpiParams ep2 = {p.bias2, nullptr, p.out2, p.Cout, p.relu2};
                const uint4 none[4] = {};
#pragma unroll 1
                for (int i = 0; i < kChunksPerWarp; ++i) {
                    const int c0 = c_base + i * 32;
                    uint32_t v[32];
                    tmem_ld_32x32(t_addr + (uint32_t)(BN + i * 32), v);
                    tmem_ld_wait();
                    if (boxed) {
                        if ((i & 1) == 0) {
                            if (lane == 0) bulk_wait_group_read<0>();
                            __syncwarp();
                        }
                        if (c0 < p.Cout) epilogue_box_bf16(ep2, v, c0, stage_tile, (i & 1) * 4, lane);
                        if (i & 1) {
                            fence_proxy_async_shared();
                            __syncwarp();
                            if (lane == 0 && c0 < p.Cout && n < p.N) {
                                tma_store_4d(&p.tmOut2, stage_tile, c0 - 32, ow, oh, n);
                                bulk_commit_group();
                            }
                        }
                    } else if (c0 < p.Cout) {
                        epilogue_coalesced_bf16<32>(ep2, v, c0, stage_tile, lane, rows, none, false);
                    }
                }
            }
          }  // pixel tiles of the work item
            if (!alive) break;
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if constexpr (kPair) mbar_arrive_cluster(map_to_cta(smem_u32(&bar_acc_empty[acc]), 0));
                else mbar_arrive(smem_u32(&bar_acc_empty[acc]));
            }
            if (++acc == kBufs) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
        if (boxed && lane == 0) bulk_wait_group_all();  // the stores have read shared memory and written the output
    }

    // ------------------------------ teardown ------------------------------
    if (*abort_ptr) {
        // Loads that were already issued may still be landing in shared memory: give them time
        // (bounded) before the CTA's shared memory is released.
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    // Neither CTA of a pair may release its TMEM or shared memory while the other can still signal or read it.
    if constexpr (kPair) cluster_sync_all();
    tc_fence_after_sync();
    if (warp == 1) {
        __syncwarp();
        if constexpr (kPair) tmem_dealloc_pair(tmem_base, kTmemCols);
        else tmem_dealloc(tmem_base, kTmemCols);
    }
    if (threadIdx.x == 0 && *abort_ptr && p.status != nullptr) atomicExch(p.status, KXC_B200_ERR_DEVICE_WAIT);
}

template <MmaKind kKind, int KB_BYTES, int BN, int kOutMode, int kCtas, bool kDual = false, int kMT = 1>
int32_t launch_one(const TcParams& p, cudaStream_t stream) {
    using G = StageGeom<KB_BYTES, BN, kCtas, kMT>;
    auto kernel = conv_igemm_kernel<kKind, KB_BYTES, BN, kOutMode, kCtas, kDual, kMT>;
    static PerDeviceOnce smem_once;
    static std::mutex units_mu;
    static int max_units[PerDeviceOnce::kMaxDevices] = {0};  // per device: clusters of two (kCtas = 2) resident at once
    int dev = 0;
    KXC_TRY(smem_opt_in(smem_once, kernel, G::kSmemBytes, &dev));
    const long long m_tiles = (long long)p.tiles_w * p.tiles_h * p.tiles_n;
    const long long tiles = (long long)p.tiles_c * ((m_tiles + kCtas * kMT - 1) / (kCtas * kMT));
    if (tiles <= 0) return KXC_B200_OK;
    int units = kNumSMs;
    if constexpr (kCtas == 2) {
        std::lock_guard<std::mutex> lock(units_mu);
        if (max_units[dev] == 0) {
            cudaLaunchConfig_t lc = {};
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 2;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            lc.gridDim = dim3(kNumSMs);
            lc.blockDim = dim3(kTcThreads);
            lc.dynamicSmemBytes = G::kSmemBytes;
            lc.attrs = attr;
            lc.numAttrs = 1;
            int n = 0;
            const cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kernel, &lc);
            if (e != cudaSuccess || n <= 0)
                return fail(KXC_B200_ERR_CUDA, "cudaOccupancyMaxActiveClusters: %s (%d clusters)", cudaGetErrorString(e), n);
            max_units[dev] = n < kNumSMs / 2 ? n : kNumSMs / 2;
        }
        units = max_units[dev];
    }
    const int grid = kCtas * (int)(tiles < units ? tiles : units);
    KXC_CUDA_TRY(launch_kernel(kernel, dim3(grid), dim3(kTcThreads), G::kSmemBytes, stream, /*pdl=*/true, kCtas, p));
    return check_launch("conv_igemm_kernel");
}

template <MmaKind kKind, int KB_BYTES, int BN, int kCtas>
int32_t launch_by_out(const TcConfig& cfg, const TcParams& p, cudaStream_t s) {
    if constexpr (kKind == MmaKind::I8) {
        switch (cfg.out_mode) {
            case kOutNHWC_S8: return launch_one<kKind, KB_BYTES, BN, kOutNHWC_S8, kCtas>(p, s);
            case kOutNCHW_S8: return launch_one<kKind, KB_BYTES, BN, kOutNCHW_S8, kCtas>(p, s);
            default: break;
        }
    } else {
        switch (cfg.out_mode) {
            case kOutNHWC_BF16: return launch_one<kKind, KB_BYTES, BN, kOutNHWC_BF16, kCtas>(p, s);
            case kOutNHWC_F32: return launch_one<kKind, KB_BYTES, BN, kOutNHWC_F32, kCtas>(p, s);
            case kOutNCHW_F32: return launch_one<kKind, KB_BYTES, BN, kOutNCHW_F32, kCtas>(p, s);
            default: break;
        }
    }
    return fail(KXC_B200_ERR_INVALID, "tensor-core conv: output mode %d does not fit dtype %d", (int)cfg.out_mode, (int)cfg.dtype);
}

template <MmaKind kKind, int KB_BYTES>
int32_t launch_by_bn(const TcConfig& cfg, const TcParams& p, cudaStream_t s) {
    if constexpr (KB_BYTES == 128 && kKind == MmaKind::F16) {
        if (cfg.dual) {
            if ((cfg.bn != 128 && cfg.bn != 192) || cfg.ctas != 1 || cfg.out_mode != kOutNHWC_BF16 || !p.vec_ok || (p.Cout & 31) != 0)
                return fail(KXC_B200_ERR_INVALID, "tensor-core conv: the two-output kernel needs a 128- or 192-wide tile, bf16 NHWC output and aligned pointers");
            return cfg.bn == 192 ? launch_one<kKind, KB_BYTES, 192, kOutNHWC_BF16, 1, true>(p, s)
                                 : launch_one<kKind, KB_BYTES, 128, kOutNHWC_BF16, 1, true>(p, s);
        }
    }
    if (cfg.dual) return fail(KXC_B200_ERR_INVALID, "tensor-core conv: no two-output kernel for this configuration");
    if constexpr (KB_BYTES == 128 && kKind == MmaKind::F16) {
        if (cfg.mt == 2) {
            if (cfg.bn != 128 || cfg.out_mode != kOutNHWC_BF16)
                return fail(KXC_B200_ERR_INVALID, "tensor-core conv: two pixel tiles per work item exist for the 128-wide bf16 NHWC kernel");
            return cfg.ctas == 2 ? launch_one<kKind, KB_BYTES, 128, kOutNHWC_BF16, 2, false, 2>(p, s)
                                 : launch_one<kKind, KB_BYTES, 128, kOutNHWC_BF16, 1, false, 2>(p, s);
        }
    }
    if (cfg.mt != 1) return fail(KXC_B200_ERR_INVALID, "tensor-core conv: no multi-tile kernel for this configuration");
    if constexpr (KB_BYTES == 128) {
        if (cfg.ctas == 2) {  // pairs exist for the wide tiles only (tc_setup_conv)
            switch (cfg.bn) {
                case 128: return launch_by_out<kKind, KB_BYTES, 128, 2>(cfg, p, s);
                case 256: return launch_by_out<kKind, KB_BYTES, 256, 2>(cfg, p, s);
                default: return fail(KXC_B200_ERR_INVALID, "tensor-core conv: no CTA-pair kernel for N tile %d", cfg.bn);
            }
        }
    }
    if (cfg.ctas != 1) return fail(KXC_B200_ERR_INVALID, "tensor-core conv: no CTA-pair kernel for %d-byte K blocks", KB_BYTES);
    switch (cfg.bn) {
        case 64: return launch_by_out<kKind, KB_BYTES, 64, 1>(cfg, p, s);
        case 128: return launch_by_out<kKind, KB_BYTES, 128, 1>(cfg, p, s);
        case 192:
            if constexpr (KB_BYTES == 128) return launch_by_out<kKind, KB_BYTES, 192, 1>(cfg, p, s);
            return fail(KXC_B200_ERR_INVALID, "tensor-core conv: the 192-wide tile exists for 128-byte K blocks only");
        case 256: return launch_by_out<kKind, KB_BYTES, 256, 1>(cfg, p, s);
        default: return fail(KXC_B200_ERR_INVALID, "tensor-core conv: unsupported N tile %d", cfg.bn);
    }
}

template <MmaKind kKind>
int32_t launch_by_kb(const TcConfig& cfg, const TcParams& p, cudaStream_t s) {
    switch (cfg.kb_bytes) {
        case 32: return launch_by_bn<kKind, 32>(cfg, p, s);
        case 64: return launch_by_bn<kKind, 64>(cfg, p, s);
        case 128: return launch_by_bn<kKind, 128>(cfg, p, s);
        default: return fail(KXC_B200_ERR_INVALID, "tensor-core conv: unsupported K block of %d bytes", cfg.kb_bytes);
    }
}

}  // namespace

int32_t tc_launch(const TcConfig& cfg, const TcParams& p, cudaStream_t stream) {
    switch (cfg.dtype) {
        case kTcBF16: return launch_by_kb<MmaKind::F16>(cfg, p, stream);
        case kTcTF32: return launch_by_kb<MmaKind::TF32>(cfg, p, stream);
        case kTcS8: return launch_by_kb<MmaKind::I8>(cfg, p, stream);
    }
    return fail(KXC_B200_ERR_INVALID, "tensor-core conv: unknown dtype");
}

void tc_pick_tile(int N, int OH, int OW, int* BW, int* BH, int* BNI) {
    double best = -1.0;
    int bw_best = 1, bh_best = 1, bn_best = 1;
    for (int bw = 1; bw <= OW && bw <= 128; ++bw) {
        for (int bh = 1; bh <= OH && bw * bh <= 128; ++bh) {
            int bn = 128 / (bw * bh);
            if (bn > N) bn = N;
            if (bn > 128) bn = 128;
            if (bn < 1) bn = 1;
            const long long tiles = (long long)((OW + bw - 1) / bw) * ((OH + bh - 1) / bh) * ((N + bn - 1) / bn);
            const double eff = (double)N * OH * OW / ((double)tiles * 128.0);
            // prefer higher efficiency; on ties the box with the most pixels per image (neighbouring filter
            // taps of one tile then re-read the same cache lines), then the squarer one (smaller halo)
            const int area = bw * bh, area_best = bw_best * bh_best;
            const int skew = bw > bh ? bw - bh : bh - bw, skew_best = bw_best > bh_best ? bw_best - bh_best : bh_best - bw_best;
            if (eff > best + 1e-9 || (eff > best - 1e-9 && (area > area_best || (area == area_best && skew < skew_best)))) {
                best = eff;
                bw_best = bw; bh_best = bh; bn_best = bn;
            }
        }
    }
    *BW = bw_best; *BH = bh_best; *BNI = bn_best;
}

int32_t tc_make_tmap(CUtensorMap* out, TcDType dtype, int rank, void* base, const uint64_t* dims,
                     const uint64_t* strides_bytes, const uint32_t* box, int swizzle_bytes) {
    static PFN_cuTensorMapEncodeTiled_v12000 encode = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    });
    if (!encode) return fail(KXC_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const CUtensorMapDataType dt = dtype == kTcBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                    : (dtype == kTcTF32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8);
    const CUtensorMapSwizzle sw = swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                                       : (swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    cuuint64_t gdims[5];
    cuuint64_t gstrides[4];
    cuuint32_t gbox[5];
    cuuint32_t estr[5];
    for (int i = 0; i < rank; ++i) {
        gdims[i] = dims[i];
        gbox[i] = box[i];
        estr[i] = 1;
        if (i + 1 < rank) gstrides[i] = strides_bytes[i];
    }
    const CUresult r = encode(out, dt, (cuuint32_t)rank, base, gdims, gstrides, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return fail(KXC_B200_ERR_CUDA,
                    "cuTensorMapEncodeTiled failed (%d): rank %d dims [%llu,%llu,%llu,%llu] box [%u,%u,%u,%u] stride0 %llu", (int)r,
                    rank, (unsigned long long)dims[0], (unsigned long long)(rank > 1 ? dims[1] : 0),
                    (unsigned long long)(rank > 2 ? dims[2] : 0), (unsigned long long)(rank > 3 ? dims[3] : 0), box[0],
                    rank > 1 ? box[1] : 0, rank > 2 ? box[2] : 0, rank > 3 ? box[3] : 0,
                    (unsigned long long)(rank > 1 ? strides_bytes[0] : 0));
    }
    return KXC_B200_OK;
}

int32_t tc_status_word(int** out) {
    static std::mutex mu;
    static int* words[64] = {nullptr};
    int dev = 0;
    KXC_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(KXC_B200_ERR_INVALID, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!words[dev]) {
        KXC_CUDA_TRY(cudaMalloc(&words[dev], sizeof(int)));
        KXC_CUDA_TRY(cudaMemset(words[dev], 0, sizeof(int)));
    }
    *out = words[dev];
    return KXC_B200_OK;
}

int32_t tc_bind_store(TcParams* p, const TcConfig& cfg) {
    p->store_box = 0;
    static const bool enabled = [] {
        const char* e = getenv("KXC_B200_TMA_STORE");
        return !(e != nullptr && e[0] == '0');
    }();
    auto pow2 = [](int v) { return v > 0 && (v & (v - 1)) == 0; };
    if (!enabled || cfg.dtype != kTcBF16 || cfg.out_mode != kOutNHWC_BF16 || cfg.bn < 128 || cfg.bn == 192 || p->out == nullptr || (p->Cout & 63) != 0 ||
        !pow2(p->BW) || !pow2(p->BH) || !pow2(p->BNI) || p->BW * p->BH * p->BNI != 128 || p->BW > 32)
        return KXC_B200_OK;
    // a warp's 32 consecutive tile rows as a box of the output tensor
    const int hw = p->BW * p->BH;
    const uint32_t sub_w = (uint32_t)p->BW;
    const uint32_t sub_h = (uint32_t)(hw >= 32 ? 32 / p->BW : p->BH);
    const uint32_t sub_n = (uint32_t)(hw >= 32 ? 1 : 32 / hw);
    const uint64_t px = (uint64_t)p->Cout * 2;
    const uint64_t dims[4] = {(uint64_t)p->Cout, (uint64_t)p->OW, (uint64_t)p->OH, (uint64_t)p->N};
    const uint64_t strides[3] = {px, (uint64_t)p->OW * px, (uint64_t)p->OH * p->OW * px};
    const uint32_t box[4] = {64u, sub_w, sub_h, sub_n};
    KXC_TRY(tc_make_tmap(&p->tmOut, kTcBF16, 4, p->out, dims, strides, box, 128));
    if (cfg.dual) {
        if (p->out2 == nullptr) return KXC_B200_OK;
        KXC_TRY(tc_make_tmap(&p->tmOut2, kTcBF16, 4, p->out2, dims, strides, box, 128));
    }
    p->store_box = 1;
    return KXC_B200_OK;
}

bool tc_dual_applicable(TcDType dtype, TcOutMode out_mode, int cpad, int Cout, int KH, int KW, int stride, int pad_h, int pad_w,
                        int dil_h, int dil_w) {
    // the second output's only tap must be the main filter's centre tap
    return dtype == kTcBF16 && out_mode == kOutNHWC_BF16 && (cpad * 2) % 128 == 0 && Cout % 32 == 0 && (KH & 1) && (KW & 1) &&
           dil_h == 1 && dil_w == 1 && pad_h == KH / 2 && pad_w == KW / 2 && (stride == 1 || stride == 2);
}

int32_t tc_setup_dual(TcParams* p, TcConfig* cfg, const void* act_nhwc, const void* w_packed, const void* w2_packed, int N,
                      int H, int W, int cpad, int Cout, int KH, int KW, int stride, int pad_h, int pad_w) {
    KXC_TRY(tc_setup_conv(p, cfg, kTcBF16, kOutNHWC_BF16, act_nhwc, w_packed, N, H, W, cpad, Cout, KH, KW, stride, pad_h, pad_w, 1, 1));
    // The two accumulators of a buffer share TMEM: 128-wide tiles (two buffers of 2 x 128 columns), single CTAs. When
    // that leaves a launch with a second, mostly empty wave and 192-wide tiles fit one wave (256 -> 512 channels at 128
    // images: 196 tiles against 147 for 148 SMs), the 192-wide form is taken: one buffer of 2 x 192 columns, so the
    // epilogue no longer overlaps the next item's MMAs, which a CTA with a single work item does not miss.
    int bn = 128;
    {
        const long long m_tiles = (long long)p->tiles_w * p->tiles_h * p->tiles_n;
        auto waves = [](long long items) { return (items + kNumSMs - 1) / kNumSMs; };
        const long long t128 = m_tiles * ((Cout + 127) / 128), t192 = m_tiles * ((Cout + 191) / 192);
        static const bool model = [] { const char* e = getenv("KXC_B200_TILE_MODEL"); return !(e != nullptr && e[0] == '0'); }();
        if (model && p->kb_elems * 2 == 128 && waves(t192) == 1 && waves(t128) >= 2) bn = 192;  // (192-wide tiles need 128-byte K blocks)
    }
    cfg->bn = bn; cfg->ctas = 1; cfg->dual = 1;
    p->tiles_c = (Cout + bn - 1) / bn;
    const uint64_t ktot = (uint64_t)KH * KW * cpad;
    const uint64_t bdims[2] = {ktot, (uint64_t)Cout};
    const uint64_t bstrides[1] = {ktot * 2};
    const uint32_t bbox[2] = {(uint32_t)p->kb_elems, (uint32_t)bn};
    KXC_TRY(tc_make_tmap(&p->tmB, kTcBF16, 2, const_cast<void*>(w_packed), bdims, bstrides, bbox, 128));
    const uint64_t b2dims[2] = {(uint64_t)cpad, (uint64_t)Cout};
    const uint64_t b2strides[1] = {(uint64_t)cpad * 2};
    KXC_TRY(tc_make_tmap(&p->tmB2, kTcBF16, 2, const_cast<void*>(w2_packed), b2dims, b2strides, bbox, 128));
    return KXC_B200_OK;
}

int32_t tc_setup_conv(TcParams* p, TcConfig* cfg, TcDType dtype, TcOutMode out_mode, const void* act_nhwc,
                      const void* w_packed, int N, int H, int W, int cpad, int Cout, int KH, int KW, int stride, int pad_h,
                      int pad_w, int dil_h, int dil_w, int* status_word) {
    const int eb = tc_elem_bytes(dtype);
    if (stride != 1 && stride != 2) return fail(KXC_B200_ERR_UNSUPPORTED, "tensor-core conv: stride %d", stride);
    const int row_bytes = cpad * eb;
    int kb_bytes;
    if (row_bytes == 32 || row_bytes == 64) kb_bytes = row_bytes;
    else if (row_bytes % 128 == 0) kb_bytes = 128;
    else return fail(KXC_B200_ERR_INVALID, "tensor-core conv: %d padded channels x %d bytes is not a K-block multiple", cpad, eb);
    const int OH = (int)conv_out_dim(H, KH, stride, pad_h, dil_h);
    const int OW = (int)conv_out_dim(W, KW, stride, pad_w, dil_w);
    if (OH <= 0 || OW <= 0) return fail(KXC_B200_ERR_INVALID, "tensor-core conv: empty output");

    p->N = N; p->OH = OH; p->OW = OW; p->Cout = Cout;
    p->taps_h = KH; p->taps_w = KW; p->stride = stride;
    p->pad_h = pad_h; p->pad_w = pad_w; p->dil_h = dil_h; p->dil_w = dil_w;
    p->kb_elems = kb_bytes / eb;
    p->cblocks = row_bytes / kb_bytes;
    tc_pick_tile(N, OH, OW, &p->BW, &p->BH, &p->BNI);
    p->tiles_w = (OW + p->BW - 1) / p->BW;
    p->tiles_h = (OH + p->BH - 1) / p->BH;
    p->tiles_n = (N + p->BNI - 1) / p->BNI;

    int bn = Cout <= 64 ? 64 : (Cout <= 128 ? 128 : 256);
    // A launch with a handful of tiles (the dense layer of a small batch: 1 pixel tile x 4 channel tiles) is bound by
    // the latency of each CTA's own operand stream: narrower tiles spread the weight rows over more SMs.
    {
        const long long mt = (long long)p->tiles_w * p->tiles_h * p->tiles_n;
        while (bn > 64 && mt * ((Cout + bn - 1) / bn) < 32) bn /= 2;
    }
    // CTA pairs (tcgen05 cta_group::2): each CTA fetches half of the B tile, which relieves the L2 -> shared-memory
    // fill rate that bounds the wide tiles. KXC_B200_CTA_PAIR=0 switches them off (for measurements).
    static const bool pair_enabled = [] {
        const char* e = getenv("KXC_B200_CTA_PAIR");
        return !(e != nullptr && e[0] == '0');
    }();
    const long long m_tiles = (long long)p->tiles_w * p->tiles_h * p->tiles_n;
    // Measured: pairs gain 5-7 % with the 256-wide tile and lose 3-10 % with the 128-wide one (the pair's MMA is
    // no faster there and the handshakes cross SMs), so only the 256-wide tile uses them. "2" forces them for 128 too.
    static const bool pair_all = [] { const char* e = getenv("KXC_B200_CTA_PAIR"); return e != nullptr && e[0] == '2'; }();
    int ctas = (pair_enabled && bn >= (pair_all ? 128 : 256) && kb_bytes == 128 && m_tiles >= 2) ? 2 : 1;
    // Launches with few tiles (small per-GPU batches in the deep layers): the 256-wide tile leaves SMs idle, e.g. 98 tiles
    // (49-50 pairs) on 148 SMs. 512 channels in 192-wide tiles on 49 pixel tiles are 147 CTAs, one wave, and an
    // M = 128, K = 16 instruction takes ~99 cycles at N = 192 against ~131 at N = 256 (measured). The narrower tile is
    // taken when the modelled makespan (waves x cycles per instruction) gains 10 %: layer 4 at 128 / 256 images per GPU
    // 37 -> 35 / 61 -> 57 us. (A 128-wide tile was measured slower there, 38 -> 45 us: without the pair's halved weight
    // fetch each CTA's operand stream from L2 becomes the limit.) KXC_B200_TILE_MODEL=0 keeps the widest tile.
    static const bool tile_model = [] {
        const char* e = getenv("KXC_B200_TILE_MODEL");
        return !(e != nullptr && e[0] == '0');
    }();
    if (tile_model && bn == 256 && kb_bytes == 128 && (dtype == kTcBF16 || dtype == kTcS8)) {
        auto waves = [](long long items, long long slots) { return (items + slots - 1) / slots; };
        const long long span256 = ctas == 2 ? waves(((m_tiles + 1) / 2) * ((Cout + 255) / 256), kNumSMs / 2) * 131
                                            : waves(m_tiles * ((Cout + 255) / 256), kNumSMs) * 131;
        const long long span192 = waves(m_tiles * ((Cout + 191) / 192), kNumSMs) * 99;
        int pick = 256;
        if (span192 * 10 <= span256 * 9) pick = 192;
        if (pick != 256) {
            bn = pick;
            ctas = 1;
        }
    }
    cfg->dtype = dtype; cfg->kb_bytes = kb_bytes; cfg->bn = bn; cfg->out_mode = out_mode; cfg->ctas = ctas;
    // Two pixel tiles per work item for the 128-wide bf16 tile: measured 0.285/0.277/0.284 -> 0.231/0.221/0.234 ms on the
    // 128->128 layers (the tensor core then sits on its operand-fetch bound: 8 KB per instruction at ~64 B/clk). With the
    // 256-wide tile TMEM holds only one buffer of two accumulators and the lost epilogue overlap costs more than the
    // second chain brings (0.168 -> 0.211 ms), so that form is not instantiated. KXC_B200_MT=1 switches it off.
    static const bool mt_enabled = [] {
        const char* e = getenv("KXC_B200_MT");
        return !(e != nullptr && e[0] == '1');
    }();
    cfg->mt = (mt_enabled && bn == 128 && dtype == kTcBF16 && out_mode == kOutNHWC_BF16 && kb_bytes == 128 && m_tiles >= 2 * ctas) ? 2 : 1;
    p->tiles_c = (Cout + bn - 1) / bn;

    const uint32_t box[4] = {(uint32_t)p->kb_elems, (uint32_t)p->BW, (uint32_t)p->BH, (uint32_t)p->BNI};
    uint8_t* base = const_cast<uint8_t*>(static_cast<const uint8_t*>(act_nhwc));
    if (stride == 1) {
        const uint64_t dims[4] = {(uint64_t)cpad, (uint64_t)W, (uint64_t)H, (uint64_t)N};
        const uint64_t strides[3] = {(uint64_t)row_bytes, (uint64_t)W * row_bytes, (uint64_t)H * W * row_bytes};
        KXC_TRY(tc_make_tmap(&p->tmA[0], dtype, 4, base, dims, strides, box, kb_bytes));
        for (int i = 1; i < 4; ++i) p->tmA[i] = p->tmA[0];
    } else {
        // One map per (row parity, column parity): the stride-2 walk over the input becomes a unit-stride
        // walk over the pixels of one parity class.
        for (int hp = 0; hp < 2; ++hp)
            for (int wp = 0; wp < 2; ++wp) {
                const int hc = (H - hp + 1) / 2, wc = (W - wp + 1) / 2;
                CUtensorMap* m = &p->tmA[hp * 2 + wp];
                if (hc <= 0 || wc <= 0)
                    return fail(KXC_B200_ERR_UNSUPPORTED, "tensor-core conv: stride 2 over a %dx%d input", H, W);
                const uint64_t dims[4] = {(uint64_t)cpad, (uint64_t)wc, (uint64_t)hc, (uint64_t)N};
                const uint64_t strides[3] = {(uint64_t)2 * row_bytes, (uint64_t)2 * W * row_bytes, (uint64_t)H * W * row_bytes};
                KXC_TRY(tc_make_tmap(m, dtype, 4, base + ((size_t)hp * W + wp) * row_bytes, dims, strides, box, kb_bytes));
            }
    }
    const uint64_t ktot = (uint64_t)KH * KW * cpad;
    const uint64_t bdims[2] = {ktot, (uint64_t)Cout};
    const uint64_t bstrides[1] = {ktot * eb};
    const uint32_t bbox[2] = {(uint32_t)p->kb_elems, (uint32_t)(bn / ctas)};
    KXC_TRY(tc_make_tmap(&p->tmB, dtype, 2, const_cast<void*>(w_packed), bdims, bstrides, bbox, kb_bytes));
    if (status_word != nullptr) {
        p->status = status_word;
    } else {
        KXC_TRY(tc_status_word(&p->status));
    }
    return KXC_B200_OK;
}

}  // namespace kxc_b200

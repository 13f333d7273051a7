// 3x3 / stride-1 / pad-1 convolution for 128 -> 128 channel layers (bf16 NHWC): the row-stacked form of
// conv_rowstack.cu on CTA pairs, with the weights resident in shared memory.
//
// The general implicit-GEMM kernel reads every input pixel nine times (one box per filter tap) and the weights once per
// work item: at 128 channels that is ~440 KB of L2 -> shared-memory traffic per 128-pixel tile, and the measured fill
// rate of an SM (~45-50 bytes per clock with all SMs loading) is what bounds those layers (0.22-0.23 ms per launch at
// 1024 images, 1.0-1.08 PFLOP/s, the same with and without CTA pairs). Here
//
//   * a work item is (pair of pixel tiles, HALF of the output channels). The three filter rows of those 64 channels are
//     stacked along N as in conv_rowstack.cu (D_0 | D_1 | D_2 in 192 TMEM columns, summed in the epilogue by a shift of
//     one accumulator row), so a tile's input is ONE halo box (16 rows x 10 columns x 128 channels = 40 KiB) whose nine
//     shifted views are shared-memory descriptor offsets;
//   * the two CTAs of a cluster issue tcgen05.mma.cta_group::2 (M = 256: each CTA's own tile; N = 192: each CTA holds
//     96 of the 192 stacked weight rows), so the 3 x 3 x 128 x 64 weights of the half cost 72 KiB per CTA and stay
//     resident for the whole launch. A pair works on one half for its lifetime (even pairs the first 64 channels, odd
//     pairs the rest); every halo is therefore fetched by two pairs (80 KiB per tile against ~440 KiB before);
//   * per work item 24 instructions (3 tap columns x 8 K slices of 16 channels), each fetching 4 KiB of A and 3 KiB of B
//     per CTA.
//
// Roles per CTA as in conv_rowstack.cu (warp 0 producer, warp 1 MMA issuer -- the leader CTA's only -- and TMEM owner,
// warps 2..17 epilogue with TMA-loaded residual boxes and TMA-stored output boxes of 64 channels); pair protocol as in
// conv_tc.cu (loads of both CTAs count on the leader's barriers, commits arrive on both CTAs' barriers, the peer's epilogue
// warps release accumulators on the leader's barrier). Every wait is bounded. No multicast loads.
#include "conv_rowstack.cuh"

#include <mutex>

#include "common.cuh"
#include "conv_epilogue.cuh"
#include "sm100.cuh"

namespace kxc_b200 {
namespace {

using namespace sm100;

// Eight epilogue warps: warp (quad, g) takes TMEM lanes [32 quad, 32 quad + 32) and the kCh = 32 channels
// [32 g, 32 g + 32) of D_0, D_1 and D_2 in ONE round of loads (96 registers), after which the accumulator goes back to
// the tensor core. Measured alternatives, all slower: sixteen warps x 16 channels (0.193 / 0.246 ms per launch without /
// with residual at 1024 images against 0.191 / 0.235), two passes of 16 channels per thread, which hold the accumulator
// through the first pass's arithmetic (0.27 ms), and two sets of eight warps, one per accumulator (0.219 ms).
constexpr int kEpiWarps = 8;
constexpr int kCh = 64 / (kEpiWarps / 4);
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kThreads = 64 + kEpiThreads;
constexpr int kC = 128;               // input channels: two planes of 64 (128-byte rows)
constexpr int kO = 128;               // output channels, in two halves of kOH
constexpr int kOH = 64;
constexpr int kBN = 3 * kOH;          // MMA N: the three filter rows of one half side by side
constexpr int kTileW = 8;
constexpr int kRows = 16;
constexpr int kOutRows = kRows - 2;
constexpr int kHaloW = kTileW + 2;
constexpr int kPlaneBytes = kHaloW * kRows * 128;   // 20480: one 64-channel plane of a halo
constexpr int kHaloBytes = 2 * kPlaneBytes;         // 40960
constexpr int kBRows = kBN / 2;                     // 96 stacked weight rows per CTA
constexpr int kWBlockBytes = kBRows * 128;          // 12288: one (tap column, plane) block of this CTA's rows
constexpr int kWeightBytes = 3 * 2 * kWBlockBytes;  // 73728
constexpr int kStages = 2;
constexpr int kAccStride = 256;
constexpr int kBoxBytes = kTileW * kOutRows * 128;  // 14336: 8 x 14 pixels x 64 channels
constexpr int kResBufs = 2;
constexpr int kOutBufs = 2;
constexpr int kSmemBytes = kWeightBytes + kStages * kHaloBytes + (kResBufs + kOutBufs) * kBoxBytes + 1024;
static_assert(kSmemBytes <= 227 * 1024, "shared memory of one CTA");

template <int kN>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&v)[kN]) {
    static_assert(kN == 32 || kN == 16, "32 or 16 columns per load");
    if constexpr (kN == 32) tmem_ld_32x32(taddr, v);
    else tmem_ld_32x16(taddr, v);
}

__global__ void __launch_bounds__(kThreads, 1) conv3x3_rowstack128_kernel(const __grid_constant__ TcParams p) {
    constexpr uint32_t kTmemCols = 2 * kAccStride;
    constexpr uint32_t kIdesc = make_instr_desc(kFmtBF16, kAccF32, kBN, 256u);

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
    const uint32_t cta_rank = cluster_cta_rank();
    const bool leader = cta_rank == 0;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar_w), 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bar_acc_full[a]), 1);
            mbar_init(smem_u32(&bar_acc_empty[a]), 2 * kEpiWarps);  // one arrival per epilogue warp of both CTAs
        }
        for (int b = 0; b < kResBufs; ++b) {
            mbar_init(smem_u32(&bar_res_full[b]), 1);
            mbar_init(smem_u32(&bar_res_empty[b]), kEpiWarps);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(&tmem_base_slot), kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers are initialised before anything signals them
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int* abort_ptr = &abort_flag;
    pdl_launch_dependents();

    // Work split: pair q of Q (Q even) works on channel half q & 1 and on the tile pairs q/2, q/2 + Q/2, ...; CTA `rank`
    // of the pair takes tile 2 * tile_pair + rank. A tile index beyond the last tile loads zeros and stores nothing.
    const int total_tiles = p.tiles_w * p.tiles_h * p.tiles_n;
    const int tile_pairs = (total_tiles + 1) >> 1;
    const int pair_id = (int)(blockIdx.x >> 1);
    const int half = pair_id & 1;
    const int first_tp = pair_id >> 1;
    const int tp_step = (int)(gridDim.x >> 2);

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&p.tmA[0]);
            tma_prefetch_desc(&p.tmB);
            if (has_res) tma_prefetch_desc(&p.tmA[1]);
            // Resident weights: this CTA's 96 of the half's 192 stacked rows (filter row r, channel co -> row 64 r + co),
            // for each tap column and channel plane, as three boxes of 32 rows. Both CTAs' bytes count on the leader's barrier.
            const uint32_t wbar = map_to_cta(smem_u32(&bar_w), 0);
            if (leader) mbar_arrive_expect_tx(smem_u32(&bar_w), 2u * kWeightBytes);
            for (int kw = 0; kw < 3; ++kw)
                for (int pl = 0; pl < 2; ++pl)
                    for (int j = 0; j < 3; ++j) {
                        const int s0 = (int)cta_rank * kBRows + 32 * j;  // first stacked row of the box
                        const int r = s0 / kOH, co0 = s0 % kOH;
                        tma_load_2d_pair(w_smem + (uint32_t)((kw * 2 + pl) * kWBlockBytes + 32 * j * 128), &p.tmB, wbar,
                                         (r * 3 + kw) * kC + pl * 64, half * kOH + co0);
                    }
            pdl_wait();  // the weights are constants; the activations come from the previous kernel
            int stage = 0, rb = 0;
            uint32_t phase = 0, rphase = 0;
            for (int tp = first_tp; tp < tile_pairs; tp += tp_step) {
                int r = 2 * tp + (int)cta_rank;
                const int tw = r % p.tiles_w; r /= p.tiles_w;
                const int th = r % p.tiles_h;
                const int tn = r / p.tiles_h;  // = N for the missing second tile of an odd count: out of range, reads zeros
                if (!mbar_wait_bounded(smem_u32(&bar_empty[stage]), phase ^ 1u, abort_ptr)) break;
                const uint32_t full = smem_u32(&bar_full[stage]);
                if (leader) mbar_arrive_expect_tx(full, 2u * kHaloBytes);
                const uint32_t full0 = map_to_cta(full, 0);
                const uint32_t dst = halo_smem + (uint32_t)(stage * kHaloBytes);
                // tensor map dimensions: channel, ROW, column, image
                tma_load_4d_pair(dst, &p.tmA[0], full0, 0, th * kOutRows - 1, tw * kTileW - 1, tn);
                tma_load_4d_pair(dst + kPlaneBytes, &p.tmA[0], full0, 64, th * kOutRows - 1, tw * kTileW - 1, tn);
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
                if (has_res) {  // this CTA's own residual box (its own barrier)
                    if (!mbar_wait_bounded(smem_u32(&bar_res_empty[rb]), rphase ^ 1u, abort_ptr)) break;
                    mbar_arrive_expect_tx(smem_u32(&bar_res_full[rb]), kBoxBytes);
                    tma_load_4d(res_smem + rb * kBoxBytes, &p.tmA[1], smem_u32(&bar_res_full[rb]), half * kOH, th * kOutRows, tw * kTileW, tn);
                    if (++rb == kResBufs) { rb = 0; rphase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            bool ok = mbar_wait_bounded(smem_u32(&bar_w), 0, abort_ptr);
            const uint32_t hi = desc_hi(1024, kLayoutSw128);
            const uint32_t b_lo0 = desc_lo(w_smem, 16);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            for (int tp = first_tp; ok && tp < tile_pairs; tp += tp_step) {
                if (!mbar_wait_bounded(smem_u32(&bar_acc_empty[acc]), acc_phase ^ 1u, abort_ptr)) break;
                if (!mbar_wait_bounded(smem_u32(&bar_full[stage]), phase, abort_ptr)) break;
                tc_fence_after_sync();
                const uint32_t d = tmem_base + (uint32_t)(acc * kAccStride);
                const uint32_t a_lo0 = desc_lo(halo_smem + stage * kHaloBytes, 16);
#pragma unroll
                for (int kw = 0; kw < 3; ++kw) {
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const uint32_t a_lo = a_lo0 + (uint32_t)(((k >> 2) * kPlaneBytes + kw * (kRows * 128) + (k & 3) * 32) >> 4);
                        const uint32_t b_lo = b_lo0 + (uint32_t)(((kw * 2 + (k >> 2)) * kWBlockBytes + (k & 3) * 32) >> 4);
                        umma_f16_split_pair(d, a_lo, hi, b_lo, hi, kIdesc, (kw | k) != 0 ? 1u : 0u);
                    }
                }
                umma_commit_pair(smem_u32(&bar_empty[stage]), 3);
                umma_commit_pair(smem_u32(&bar_acc_full[acc]), 3);
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
    } else {
        const int quad = warp & 3;
        const int c0 = ((warp - 2) >> 2) * kCh;  // channels [c0, c0 + kCh) of the pair's half
        const int h_l = lane & 15;              // accumulator row = input row of the tile
        const int w_l = 2 * quad + (lane >> 4);
        const bool issuer = threadIdx.x == 64;  // the epilogue thread that owns the TMA stores' async groups
        const bool in_box = (h_l >= 1) && (h_l <= kOutRows);
        const uint32_t box_row = (uint32_t)(w_l * kOutRows + (h_l - 1));
        const uint32_t row_off = box_row * 128u;
        const uint32_t sw = box_row & 7u;
        const uint32_t acc_empty0 = map_to_cta(smem_u32(&bar_acc_empty[0]), 0);
        const uint32_t acc_empty1 = map_to_cta(smem_u32(&bar_acc_empty[1]), 0);
        float bias[kCh];
#pragma unroll
        for (int j = 0; j < kCh; ++j) bias[j] = p.bias != nullptr ? __ldg(p.bias + half * kOH + c0 + j) : 0.0f;
        pdl_wait();
        int acc = 0, rb = 0, ob = 0;
        uint32_t acc_phase = 0, rphase = 0;
        for (int tp = first_tp; tp < tile_pairs; tp += tp_step) {
            int r = 2 * tp + (int)cta_rank;
            const int tw = r % p.tiles_w; r /= p.tiles_w;
            const int th = r % p.tiles_h;
            const int n = r / p.tiles_h;
            bool bad = !__all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&bar_acc_full[acc]), acc_phase, abort_ptr));
            float f[kCh];
            if (!bad) {
                tc_fence_after_sync();
                const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * kAccStride + c0);
                uint32_t v0[kCh], v1[kCh], v2[kCh];
                tmem_ld_cols(t_addr, v0);            // D_0: wanted by the row below
                tmem_ld_cols(t_addr + kOH, v1);      // D_1: this row
                tmem_ld_cols(t_addr + 2 * kOH, v2);  // D_2: wanted by the row above
                tmem_ld_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(acc ? acc_empty1 : acc_empty0);  // accumulator is in registers now
#pragma unroll
                for (int j = 0; j < kCh; ++j) {
                    const float up = __uint_as_float(__shfl_up_sync(0xffffffffu, v0[j], 1));
                    const float down = __uint_as_float(__shfl_down_sync(0xffffffffu, v2[j], 1));
                    f[j] = __fadd_rn(__fadd_rn(__fadd_rn(up, __uint_as_float(v1[j])), down), bias[j]);
                }
            }
            if (has_res && !bad) {
                bad = !__all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&bar_res_full[rb]), rphase, abort_ptr));
                if (!bad) {
                    if (in_box) {
                        const uint32_t base = res_smem + rb * kBoxBytes + row_off;
#pragma unroll
                        for (int g = 0; g < kCh / 8; ++g) {
                            const uint4 rv = ld_shared_v4(base + ((((uint32_t)((c0 >> 3) + g)) ^ sw) << 4));
                            const uint32_t w[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                f[g * 8 + 2 * k] = __fadd_rn(f[g * 8 + 2 * k], bf16_lo(w[k]));
                                f[g * 8 + 2 * k + 1] = __fadd_rn(f[g * 8 + 2 * k + 1], bf16_hi(w[k]));
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bar_res_empty[rb]));
                    if (++rb == kResBufs) { rb = 0; rphase ^= 1u; }
                }
            }
            if (p.relu) {
#pragma unroll
                for (int j = 0; j < kCh; ++j) f[j] = f[j] > 0.0f ? f[j] : 0.0f;
            }
            // the output box used two tiles ago must have been read by its TMA store before it is overwritten
            if (issuer) bulk_wait_group_read<kOutBufs - 1>();
            if (named_barrier_or(1, kEpiThreads, bad)) break;
            if (in_box) {
                const uint32_t base = out_smem + ob * kBoxBytes + row_off;
#pragma unroll
                for (int g = 0; g < kCh / 8; ++g) {
                    uint4 o;
                    o.x = pack_bf16(f[g * 8 + 0], f[g * 8 + 1]);
                    o.y = pack_bf16(f[g * 8 + 2], f[g * 8 + 3]);
                    o.z = pack_bf16(f[g * 8 + 4], f[g * 8 + 5]);
                    o.w = pack_bf16(f[g * 8 + 6], f[g * 8 + 7]);
                    st_shared_v4(base + ((((uint32_t)((c0 >> 3) + g)) ^ sw) << 4), o);
                }
            }
            fence_proxy_async_shared();
            named_barrier(2, kEpiThreads);
            if (issuer) {  // pixels beyond the image's last row or column are clipped by the store
                if (n < p.N) tma_store_4d(&p.tmA[2], out_smem + ob * kBoxBytes, half * kOH, th * kOutRows, tw * kTileW, n);
                bulk_commit_group();  // (an empty group for the missing second tile keeps the group count in step)
            }
            ob ^= 1;
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1u;
        }
        if (issuer) bulk_wait_group_all();
    }

    if (*abort_ptr) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // neither CTA releases TMEM or shared memory while the other can still signal or read it
    tc_fence_after_sync();
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc_pair(tmem_base, kTmemCols);
    }
    if (threadIdx.x == 0 && *abort_ptr && p.status != nullptr) atomicExch(p.status, KXC_B200_ERR_DEVICE_WAIT);
}

}  // namespace

bool rowstack128_applicable(TcDType dtype, int C, int O, int KH, int KW, int stride, int pad_h, int pad_w, int dil_h, int dil_w) {
    return dtype == kTcBF16 && C == kC && O == kO && KH == 3 && KW == 3 && stride == 1 && pad_h == 1 && pad_w == 1 && dil_h == 1 &&
           dil_w == 1;
}

int32_t rowstack128_setup(TcParams* p, const void* act_nhwc, const void* w_packed, int N, int H, int W) {
    p->N = N; p->OH = H; p->OW = W; p->Cout = kO;
    p->taps_h = 3; p->taps_w = 3; p->stride = 1; p->pad_h = 1; p->pad_w = 1; p->dil_h = 1; p->dil_w = 1;
    p->cblocks = 2; p->kb_elems = 64;
    p->BW = kTileW; p->BH = kOutRows; p->BNI = 1;
    p->tiles_w = (W + kTileW - 1) / kTileW;
    p->tiles_h = (H + kOutRows - 1) / kOutRows;
    p->tiles_n = N;
    p->tiles_c = 2;
    const uint64_t px = kC * 2;
    // dimensions: channel, ROW, column, image -> a box lands in shared memory as [column][row][64 channels]
    const uint64_t dims[4] = {(uint64_t)kC, (uint64_t)H, (uint64_t)W, (uint64_t)N};
    const uint64_t strides[3] = {(uint64_t)W * px, px, (uint64_t)H * W * px};
    const uint32_t box[4] = {64u, (uint32_t)kRows, (uint32_t)kHaloW, 1u};
    KXC_TRY(tc_make_tmap(&p->tmA[0], kTcBF16, 4, const_cast<void*>(act_nhwc), dims, strides, box, 128));
    for (int i = 1; i < 4; ++i) p->tmA[i] = p->tmA[0];
    const uint64_t ktot = (uint64_t)9 * kC;
    const uint64_t bdims[2] = {ktot, (uint64_t)kO};
    const uint64_t bstr[1] = {ktot * 2};
    const uint32_t bbox[2] = {64u, 32u};
    KXC_TRY(tc_make_tmap(&p->tmB, kTcBF16, 2, const_cast<void*>(w_packed), bdims, bstr, bbox, 128));
    KXC_TRY(tc_status_word(&p->status));
    return KXC_B200_OK;
}

int32_t rowstack128_bind(TcParams* p) {
    // tmA[1]: residual boxes (loads), tmA[2]: output boxes (stores): 8 x 14 pixels x 64 channels of the 128
    if (p->out == nullptr) return fail(KXC_B200_ERR_INVALID, "row-stacked 128-channel conv: no output tensor");
    const uint64_t px = kO * 2;
    const uint64_t dims[4] = {(uint64_t)kO, (uint64_t)p->OH, (uint64_t)p->OW, (uint64_t)p->N};
    const uint64_t strides[3] = {(uint64_t)p->OW * px, px, (uint64_t)p->OH * p->OW * px};
    const uint32_t box[4] = {(uint32_t)kOH, (uint32_t)kOutRows, (uint32_t)kTileW, 1u};
    KXC_TRY(tc_make_tmap(&p->tmA[2], kTcBF16, 4, p->out, dims, strides, box, 128));
    if (p->residual != nullptr)
        KXC_TRY(tc_make_tmap(&p->tmA[1], kTcBF16, 4, const_cast<void*>(p->residual), dims, strides, box, 128));
    return KXC_B200_OK;
}

int32_t rowstack128_launch(const TcParams& p, cudaStream_t stream) {
    static PerDeviceOnce smem_once;
    static std::mutex units_mu;
    static int max_pairs[PerDeviceOnce::kMaxDevices] = {0};  // per device: clusters of two resident at once
    int dev = 0;
    auto kernel = conv3x3_rowstack128_kernel;
    KXC_TRY(smem_opt_in(smem_once, kernel, kSmemBytes, &dev));
    if (!p.vec_ok || p.out == nullptr) return fail(KXC_B200_ERR_INVALID, "row-stacked 128-channel conv: pointers must be 16-byte aligned");
    const long long tiles = (long long)p.tiles_w * p.tiles_h * p.tiles_n;
    if (tiles <= 0) return KXC_B200_OK;
    int pairs;
    {
        std::lock_guard<std::mutex> lock(units_mu);
        if (max_pairs[dev] == 0) {
            cudaLaunchConfig_t lc = {};
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 2;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            lc.gridDim = dim3(kNumSMs);
            lc.blockDim = dim3(kThreads);
            lc.dynamicSmemBytes = kSmemBytes;
            lc.attrs = attr;
            lc.numAttrs = 1;
            int n = 0;
            const cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kernel, &lc);
            if (e != cudaSuccess || n < 2)
                return fail(KXC_B200_ERR_CUDA, "cudaOccupancyMaxActiveClusters: %s (%d clusters)", cudaGetErrorString(e), n);
            max_pairs[dev] = (n < kNumSMs / 2 ? n : kNumSMs / 2) & ~1;  // even: one set of pairs per channel half
        }
        pairs = max_pairs[dev];
    }
    const long long tile_pairs = (tiles + 1) / 2;
    if (2 * tile_pairs < pairs) pairs = (int)(2 * tile_pairs);
    KXC_CUDA_TRY(launch_kernel(kernel, dim3(2 * pairs), dim3(kThreads), kSmemBytes, stream, /*pdl=*/true, 2, p));
    return check_launch("conv3x3_rowstack128_kernel");
}

}  // namespace kxc_b200

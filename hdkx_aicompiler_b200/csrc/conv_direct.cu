// Direct 3x3 / stride-1 / pad-1 convolution for 64 -> 64 channel layers (bf16 NHWC), on tcgen05 + TMEM.
//
// The implicit-GEMM kernel (conv_tc.cu) issues one TMA box per filter tap, so every input pixel crosses
// the crossbar nine times and the 64x576 weights are re-fetched for every tile; for a layer with only 64
// output channels the TMA row rate, not the tensor pipe or HBM, bounds it. This kernel removes both:
//
//   * the 9 x 64 x 64 weights (72 KiB, SWIZZLE_128B) are loaded ONCE per CTA and stay in shared memory;
//   * per output tile (8 columns x 16 rows of one image) the input HALO tile — 18 rows x 16 pixels x 64
//     channels, one TMA box, zero-filled outside the image — is loaded ONCE; the A operand of tap (kh, kw)
//     is that same shared memory viewed through a matrix descriptor whose start address is advanced by
//     (kh*16 + kw) pixels: 8-row groups are one halo row (16 pixels = 2048 B) apart, so each group of 8
//     consecutive output columns is 8 consecutive 128-byte pixel rows of the halo tile.
//
// The shared-memory swizzle is a function of the address (TMA writes it that way, the MMA reads it that
// way), which is what makes a view at a 128-byte-granular offset legal.
//
// Roles as in conv_tc.cu: warp 0 producer, warp 1 MMA issuer + TMEM owner, warps 2..9 epilogue; two TMEM
// accumulators; every wait bounded.
#include "conv_direct.cuh"

#include <mutex>

#include "common.cuh"
#include "conv_epilogue.cuh"
#include "sm100.cuh"

namespace kxc_b200 {
namespace {

using namespace sm100;

constexpr int kThreads = 320;
constexpr int kC = 64;                 // input channels per block = one 128-byte row
constexpr int kBN = 64;                // output channels
constexpr int kTaps = 9;
constexpr int kTileW = 8, kTileH = 16; // output tile
constexpr int kHaloW = 16, kHaloH = kTileH + 2;
constexpr int kHaloBytes = kHaloH * kHaloW * 128;  // 36864
constexpr int kWeightBytes = kTaps * kBN * 128;    // 73728
constexpr int kStages = 4;
constexpr int kAccs = 4;               // TMEM accumulators: two tiles in flight on the tensor core + two being drained
constexpr int kSmemBytes = kWeightBytes + kStages * kHaloBytes + 1024;

// Descriptors: SWIZZLE_128B, K-major, explicit 8-row-group stride (2048 B for the halo views, 1024 B for the
// weights). The descriptor's base-offset field stays 0 even when a view's start address is not 1024-byte aligned:
// measured on B200, the swizzle phase the MMA applies comes from the shared-memory address itself (a non-zero
// base offset for the shifted views gives wrong sums).
__global__ void __launch_bounds__(kThreads, 1) conv3x3_direct_kernel(const __grid_constant__ TcParams p) {
    constexpr uint32_t kTmemCols = kAccs * kBN;
    constexpr uint32_t kIdesc = make_instr_desc(kFmtBF16, kAccF32, kBN);

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_w;
    __shared__ __align__(8) uint64_t bar_full[kStages];
    __shared__ __align__(8) uint64_t bar_empty[kStages];
    __shared__ __align__(8) uint64_t bar_acc_full[kAccs];
    __shared__ __align__(8) uint64_t bar_acc_empty[kAccs];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t w_smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t halo_smem = w_smem + kWeightBytes;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar_w), 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int a = 0; a < kAccs; ++a) {
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
            // resident weights: nine 64x64 tap blocks
            mbar_arrive_expect_tx(smem_u32(&bar_w), kWeightBytes);
            for (int t = 0; t < kTaps; ++t) tma_load_2d(w_smem + t * (kBN * 128), &p.tmB, smem_u32(&bar_w), t * kC, 0);
            pdl_wait();  // the weights are constants; the activations come from the previous kernel
            int stage = 0;
            uint32_t phase = 0;
            for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
                int r = tile;
                const int tw = r % p.tiles_w; r /= p.tiles_w;
                const int th = r % p.tiles_h;
                const int tn = r / p.tiles_h;
                if (!mbar_wait_bounded(smem_u32(&bar_empty[stage]), phase ^ 1u, abort_ptr)) break;
                const uint32_t full = smem_u32(&bar_full[stage]);
                mbar_arrive_expect_tx(full, kHaloBytes);
                tma_load_4d(halo_smem + stage * kHaloBytes, &p.tmA[0], full, 0, tw * kTileW - 1, th * kTileH - 1, tn);
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = mbar_wait_bounded(smem_u32(&bar_w), 0, abort_ptr);
            const uint32_t a_hi = desc_hi(kHaloW * 128, kLayoutSw128), b_hi = desc_hi(1024, kLayoutSw128);
            const uint32_t b_lo0 = desc_lo(w_smem, 16);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            // Consecutive MMAs into ONE accumulator form a dependent chain, and at N = 64 the chain latency (about
            // twice the 32-cycle issue interval) is what bounds the kernel. Two tiles are therefore processed
            // together, their MMAs alternating between two accumulators; each tile still sees its own 36 MMAs in
            // the same order, so the sums are unchanged.
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += 2 * gridDim.x) {
                const bool pair = tile + (int)gridDim.x < total_tiles;
                const int acc1 = (acc + 1) & (kAccs - 1);
                const int stage1 = stage + 1 == kStages ? 0 : stage + 1;
                const uint32_t phase1 = stage + 1 == kStages ? phase ^ 1u : phase;
                const uint32_t acc_phase1 = acc1 == 0 ? acc_phase ^ 1u : acc_phase;
                if (!mbar_wait_bounded(smem_u32(&bar_acc_empty[acc]), acc_phase ^ 1u, abort_ptr)) break;
                if (!mbar_wait_bounded(smem_u32(&bar_full[stage]), phase, abort_ptr)) break;
                if (pair) {
                    if (!mbar_wait_bounded(smem_u32(&bar_acc_empty[acc1]), acc_phase1 ^ 1u, abort_ptr)) break;
                    if (!mbar_wait_bounded(smem_u32(&bar_full[stage1]), phase1, abort_ptr)) break;
                }
                tc_fence_after_sync();
                const uint32_t d0 = tmem_base + (uint32_t)(acc * kBN), d1 = tmem_base + (uint32_t)(acc1 * kBN);
                // descriptor low words: base of the halo stage / of the resident weights, plus compile-time offsets
                const uint32_t a0 = desc_lo(halo_smem + stage * kHaloBytes, 16), a1 = desc_lo(halo_smem + stage1 * kHaloBytes, 16);
#pragma unroll
                for (int kh = 0; kh < 3; ++kh) {
#pragma unroll
                    for (int kw = 0; kw < 3; ++kw) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint32_t a_off = (uint32_t)(((kh * kHaloW + kw) * 128 + k * 32) >> 4);
                            const uint32_t b_lo = b_lo0 + (uint32_t)((((kh * 3 + kw) * (kBN * 128)) + k * 32) >> 4);
                            const uint32_t accum = (kh | kw | k) != 0 ? 1u : 0u;
                            umma_f16_split(d0, a0 + a_off, a_hi, b_lo, b_hi, kIdesc, accum);
                            if (pair) umma_f16_split(d1, a1 + a_off, a_hi, b_lo, b_hi, kIdesc, accum);
                        }
                    }
                }
                umma_commit(smem_u32(&bar_empty[stage]));
                umma_commit(smem_u32(&bar_acc_full[acc]));
                if (pair) {
                    umma_commit(smem_u32(&bar_empty[stage1]));
                    umma_commit(smem_u32(&bar_acc_full[acc1]));
                }
                const int used = pair ? 2 : 1;
                for (int u = 0; u < used; ++u) {
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                    acc = (acc + 1) & (kAccs - 1);
                    if (acc == 0) acc_phase ^= 1u;
                }
            }
        }
    } else {
        const int quad = warp & 3;
        const int half = (warp - 2) >> 2;  // columns [32*half, 32*half+32)
        const int row = quad * 32 + lane;
        const int h_l = row >> 3, w_l = row & 7;
        const bool has_res = p.residual != nullptr;
        pdl_wait();
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            int r = tile;
            const int tw = r % p.tiles_w; r /= p.tiles_w;
            const int th = r % p.tiles_h;
            const int n = r / p.tiles_h;
            const int oh = th * kTileH + h_l, ow = tw * kTileW + w_l;
            const bool valid = (oh < p.OH) && (ow < p.OW);
            const size_t pix = ((size_t)n * p.OH + oh) * p.OW + ow;
            const int c0 = half * 32;
            uint4 res[4] = {};
            if (has_res && valid) {
                const uint4* rp = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.residual) + pix * kBN + c0);
#pragma unroll
                for (int g = 0; g < 4; ++g) res[g] = __ldg(rp + g);
            }
            bool ok = mbar_wait_bounded(smem_u32(&bar_acc_full[acc]), acc_phase, abort_ptr);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            uint32_t v[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * kBN + c0), v);
            tmem_ld_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[acc]));  // accumulator is in registers now
            if (valid) epilogue_fast_bf16(p, v, c0, pix, res, has_res);
            acc = (acc + 1) & (kAccs - 1);
            if (acc == 0) acc_phase ^= 1u;
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

bool direct3x3_applicable(TcDType dtype, int C, int O, int KH, int KW, int stride, int pad_h, int pad_w, int dil_h, int dil_w,
                          int OW) {
    return dtype == kTcBF16 && C == kC && O == kBN && KH == 3 && KW == 3 && stride == 1 && pad_h == 1 && pad_w == 1 &&
           dil_h == 1 && dil_w == 1 && (OW % kTileW) == 0;
}

int32_t direct3x3_setup(TcParams* p, const void* act_nhwc, const void* w_packed, int N, int H, int W) {
    p->N = N; p->OH = H; p->OW = W; p->Cout = kBN;
    p->taps_h = 3; p->taps_w = 3; p->stride = 1; p->pad_h = 1; p->pad_w = 1; p->dil_h = 1; p->dil_w = 1;
    p->cblocks = 1; p->kb_elems = kC;
    p->BW = kTileW; p->BH = kTileH; p->BNI = 1;
    p->tiles_w = W / kTileW;
    p->tiles_h = (H + kTileH - 1) / kTileH;
    p->tiles_n = N;
    p->tiles_c = 1;
    const uint64_t row = kC * 2;
    const uint64_t dims[4] = {(uint64_t)kC, (uint64_t)W, (uint64_t)H, (uint64_t)N};
    const uint64_t strides[3] = {row, (uint64_t)W * row, (uint64_t)H * W * row};
    const uint32_t box[4] = {(uint32_t)kC, (uint32_t)kHaloW, (uint32_t)kHaloH, 1u};
    KXC_TRY(tc_make_tmap(&p->tmA[0], kTcBF16, 4, const_cast<void*>(act_nhwc), dims, strides, box, 128));
    for (int i = 1; i < 4; ++i) p->tmA[i] = p->tmA[0];
    const uint64_t ktot = (uint64_t)kTaps * kC;
    const uint64_t bdims[2] = {ktot, (uint64_t)kBN};
    const uint64_t bstr[1] = {ktot * 2};
    const uint32_t bbox[2] = {(uint32_t)kC, (uint32_t)kBN};
    KXC_TRY(tc_make_tmap(&p->tmB, kTcBF16, 2, const_cast<void*>(w_packed), bdims, bstr, bbox, 128));
    KXC_TRY(tc_status_word(&p->status));
    return KXC_B200_OK;
}

int32_t direct3x3_launch(const TcParams& p, cudaStream_t stream) {
    static PerDeviceOnce smem_once;
    KXC_TRY(smem_opt_in(smem_once, conv3x3_direct_kernel, kSmemBytes));
    if (!p.vec_ok || p.out == nullptr) return fail(KXC_B200_ERR_INVALID, "direct 3x3 conv: pointers must be 16-byte aligned");
    const long long tiles = (long long)p.tiles_w * p.tiles_h * p.tiles_n;
    if (tiles <= 0) return KXC_B200_OK;
    const int grid = (int)(tiles < kNumSMs ? tiles : kNumSMs);
    KXC_CUDA_TRY(launch_kernel(conv3x3_direct_kernel, dim3(grid), dim3(kThreads), kSmemBytes, stream, /*pdl=*/true, 1, p));
    return check_launch("conv3x3_direct_kernel");
}

}  // namespace kxc_b200

// 7x7 stride-2 "stem" convolution + bias + ReLU + max_pool2d(3x3, stride 2, pad 1) in ONE kernel that reads the
// graph input as the reference hands it over (NCHW fp32, include/te/topi/nn.h:107-158 / :161-229) and writes the
// pooled bf16 NHWC activation: neither a packed copy of the input nor the convolution's output touches HBM.
//
// Work split of a CTA (22 warps), all roles running concurrently on a ring of input strips:
//   warp 0        loads the 28 KiB of weights once (bulk copy)
//   warps 18..21  converters: bring the fp32 rows of a strip (three channel planes) into shared memory with cp.async,
//                 one strip ahead, round to bf16 and write the packed layout [row][pixel][4 channels] (8 bytes per
//                 pixel, zero border) that the tensor core reads
//   warp 1        issues tcgen05.mma, owns TMEM
//   warps 2..17   epilogue: accumulator -> +bias -> bf16 -> running 3x3 maximum -> ReLU -> store
//
// MMA formulation. In the packed layout the K vector of output pixel (oh, ow) for filter row r is the 8 pixels x 4
// channels starting at packed pixel (2*oh + r, 2*ow): with the unswizzled K-major operand layout (rows 16 bytes
// apart) the A operand of 128 consecutive output columns is a window of ONE packed input row (conv_stem.cu). The
// older kernel issues 14 instructions of N = 64 per output row, which the tensor core cannot run faster than about
// 74 cycles each however short their math is (32 cycles). Here one instruction serves SEVERAL output rows: packed
// input row t contributes, through filter row r = t - 2j, to every output row j of a block of three for which
// 0 <= r <= 6, and these rows' accumulators lie side by side in TMEM. So the B operand of the instruction for input
// row t is the stack [W(r_max); W(r_max - 2); ...] of the filter rows of t's parity (N = 64, 128 or 192) and D spans
// the matching accumulator slots: 24 instructions per three output rows instead of 42, most of them wide enough to
// run at the tensor pipe's full rate. Input rows are walked in ascending order and each slot's first contribution
// (r = 0) is an instruction of its own with the accumulate flag off, so every output element sums its 28 K chunks in
// exactly the order the one-row-at-a-time kernel uses: the two kernels give identical bits.
//
// Pooling in the epilogue: a thread owns one convolution column's 32 channels as 16 packed bf16 pairs. The three
// convolution rows of a pooled row arrive one after the other, so the vertical maximum is a running maximum in
// registers; once per pooled row the even columns take their neighbours' values with two shuffles per register (the
// neighbour in another warp comes through a 64-byte shared-memory slot and a 128-thread barrier). Rounding to bf16
// is monotonic and keeps the sign, so max-then-ReLU on rounded values equals the reference's ReLU-then-fold
// `m = (m > v) ? m : v` (NaN -> 0, -0 -> +0 included): 0 is a neutral element and one final max with 0 is the ReLU.
// Every wait is bounded (sm100::mbar_wait_bounded); a wait that runs out is reported through the status word.
#include "conv_stem.cuh"

#include <cuda_bf16.h>

#include "common.cuh"
#include "conv_epilogue.cuh"
#include "sm100.cuh"

namespace kxc_b200 {
namespace {

using namespace sm100;

constexpr int kPartCols = 32;       // output channels per epilogue warp: 8 epilogue warps (16 warps of 16 channels starve the converters)
constexpr int kEpilogueWarp0 = 2, kEpilogueWarps = 4 * (64 / kPartCols);
constexpr int kThreads = (2 + kEpilogueWarps + 4) * 32;  // loader, MMA issuer, epilogue warps, 4 converter warps
constexpr int kBN = 64;             // output channels
constexpr int kKH = 7;
constexpr int kPooledRows = 4;      // pooled rows per strip
constexpr int kConvRows = 2 * kPooledRows + 1;             // 9: conv rows 8s-1 .. 8s+7 (the first one recomputed)
constexpr int kInRows = 2 * (kConvRows - 1) + kKH;         // 23 packed input rows
constexpr int kMaxRowBytes = 2048;
constexpr int kStripBytes = ((kInRows * kMaxRowBytes + 4096 + 1023) / 1024) * 1024;  // + slack for the M = 128 over-read
constexpr int kStages = 2;          // packed strips in shared memory (the tensor core reads one while the next is written)
constexpr int kEvenRows = 4 * kBN, kOddRows = 3 * kBN;     // stacked filter rows: r = 6,4,2,0 and r = 5,3,1
constexpr int kWeightBytes = 4 * (kEvenRows + kOddRows) * 16;  // 4 K chunks of 8 elements per filter row: 28672
constexpr int kBlockRows = 3;       // output rows per accumulator buffer
constexpr int kBufCols = 256;       // TMEM columns per buffer (3 slots of 64 used)
constexpr int kMaxEntries = 24;     // MMA instructions of a three-row block
constexpr int kExchBytes = 2 * (64 / kPartCols) * 4 * kPartCols * 2;  // [parity][channel part][quadrant] x one column's channels of the part
constexpr int kConverterWarp0 = kEpilogueWarp0 + kEpilogueWarps, kConverterThreads = 128;
// fp32 staging of ONE strip, filled by cp.async: every converter thread owns the 16-byte slots of its own 4-pixel items
// ([item][channel][thread]), so no thread ever waits for another one's copies
constexpr int kMaxC = 3;
constexpr int kMaxRowItems = kMaxRowBytes / 32;                                                        // 4-pixel items per row
constexpr int kItemsPerThread = (kInRows * 56 + kConverterThreads - 1) / kConverterThreads;            // 11 for 224-pixel rows
constexpr int kStagingBytes = kItemsPerThread * kMaxC * kConverterThreads * 16;                          // 67584
constexpr int kSmemBytes = kWeightBytes + kStages * kStripBytes + kExchBytes + kStagingBytes + 1024;

// The instruction list of a block of R output rows (see the file comment), built at compile time so that the issue
// loop is straight-line code with immediate operands: a single thread can then issue an MMA every ~25 cycles. (A loop
// that fetches its operands from a table costs ~140 cycles per instruction in the one issuing thread, twice what the
// tensor core needs for the instruction itself.)
struct MmaEntry {
    int t, cp;        // packed input row relative to the block's first one; which pair of K chunks
    uint32_t b_rel;   // low descriptor word of the stacked weights, relative to the weights' base address
    int d_off, n, acc;
};
struct MmaTable {
    MmaEntry e[kMaxEntries];
    int len;
};
__host__ __device__ constexpr MmaTable make_mma_table(int R) {
    MmaTable tb{};
    int n = 0;
    for (int t = 0; t <= 2 * (R - 1) + (kKH - 1); ++t) {
        const int jmin = t > kKH - 1 ? (t - (kKH - 1) + 1) / 2 : 0;
        const int jmax = (t / 2) < (R - 1) ? (t / 2) : (R - 1);
        const int odd = t & 1;
        const int r_first = t - 2 * jmin;  // filter row of the first (lowest) slot: the largest of the range
        const int q = odd ? (kKH - 2 - r_first) / 2 : (kKH - 1 - r_first) / 2;
        const int cnt = jmax - jmin + 1;
        const uint32_t lbo = (uint32_t)(odd ? kOddRows : kEvenRows) * 16u;
        const uint32_t wbase = (odd ? 4u * kEvenRows * 16u : 0u) + (uint32_t)q * kBN * 16u;
        for (int cp = 0; cp < 2; ++cp) {
            const uint32_t b_addr = wbase + (uint32_t)cp * 2u * lbo;
            const uint32_t lbo_field = (lbo >> 4) << 16;
            const bool first_touch = cp == 0 && !odd && t == 2 * jmax;  // slot jmax receives filter row 0 here
            if (first_touch) {
                if (cnt > 1) tb.e[n++] = MmaEntry{t, cp, (b_addr >> 4) | lbo_field, jmin * kBN, (cnt - 1) * kBN, 1};
                tb.e[n++] = MmaEntry{t, cp, ((b_addr + (uint32_t)(cnt - 1) * kBN * 16u) >> 4) | lbo_field, jmax * kBN, kBN, 0};
            } else {
                tb.e[n++] = MmaEntry{t, cp, (b_addr >> 4) | lbo_field, jmin * kBN, cnt * kBN, 1};
            }
        }
    }
    tb.len = n;
    return tb;
}

template <int kAcc>
__device__ __forceinline__ void umma_f16_imm(uint32_t d_tmem, uint32_t a_lo, uint32_t hi, uint32_t b_lo, uint32_t idesc) {
    // both descriptors share the upper word (unswizzled, 8-row groups 128 B apart); the accumulate flag is an immediate
    if constexpr (kAcc != 0) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.eq.u32 p, 1, 1;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %2};\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(d_tmem), "r"(a_lo), "r"(hi), "r"(b_lo), "r"(idesc)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.eq.u32 p, 1, 0;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %2};\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(d_tmem), "r"(a_lo), "r"(hi), "r"(b_lo), "r"(idesc)
            : "memory");
    }
}

template <int R, int I = 0>
__device__ __forceinline__ void issue_block(uint32_t d0, uint32_t a_lo0, uint32_t row16, uint32_t hi, uint32_t w_lo) {
    constexpr MmaTable tb = make_mma_table(R);
    if constexpr (I < tb.len) {
        constexpr MmaEntry e = tb.e[I];
        constexpr uint32_t idesc = make_instr_desc(kFmtBF16, kAccF32, (uint32_t)e.n);
        umma_f16_imm<e.acc>(d0 + (uint32_t)e.d_off, a_lo0 + (uint32_t)e.t * row16 + (uint32_t)(e.cp * 2), hi, w_lo + e.b_rel, idesc);
        issue_block<R, I + 1>(d0, a_lo0, row16, hi, w_lo);
    }
}

__device__ __forceinline__ void tmem_ld_part(uint32_t taddr, uint32_t (&v)[32]) { tmem_ld_32x32(taddr, v); }

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}

__global__ void __launch_bounds__(kThreads, 1) conv_stem_pool_nchw_kernel(const __grid_constant__ TcParams p) {
    constexpr uint32_t kTmemCols = 2 * kBufCols;

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_w;
    __shared__ __align__(8) uint64_t bar_full[kStages];
    __shared__ __align__(8) uint64_t bar_empty[kStages];
    __shared__ __align__(8) uint64_t bar_acc_full[2];
    __shared__ __align__(8) uint64_t bar_acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t w_smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t strip_smem = w_smem + kWeightBytes;
    const uint32_t exch_smem = strip_smem + kStages * kStripBytes;
    const uint32_t staging_smem = exch_smem + kExchBytes;

    const int row_bytes = p.aux_row_bytes;  // packed row: Wp * 8
    const int Hp = p.aux_hp;
    const int H = p.aux_h, W = p.aux_w_px, C = p.aux_c;
    const int strips_per_image = p.OH / (2 * kPooledRows);
    const int total_strips = strips_per_image * p.N;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar_w), 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), kConverterThreads / 32);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bar_acc_full[a]), 1);
            mbar_init(smem_u32(&bar_acc_empty[a]), kEpilogueWarps);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
        tmem_relinquish();
    }
    // Zero borders and slack: the converters only ever write the pixels of the image; the MMA of the last output
    // columns reads a little past a row's end (finite values that feed accumulator rows nobody stores).
    for (uint32_t i = threadIdx.x; i < (uint32_t)(kStages * kStripBytes / 16); i += kThreads) {
        const uint32_t addr = strip_smem + i * 16;
        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
    }
    fence_proxy_async_shared();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int* abort_ptr = &abort_flag;
    pdl_launch_dependents();

    // Strip s of an image: conv rows 8s-1 .. 8s+7 (local j = 0..8; j = 0 is skipped for s = 0, it is the pool's padding
    // row), packed input rows from max(16s - 2, 0); blocks of up to three conv rows.
    if (warp == 0) {
        if (lane == 0) {
            mbar_arrive_expect_tx(smem_u32(&bar_w), (uint32_t)kWeightBytes);
            bulk_copy_g2s(w_smem, p.aux_w, (uint32_t)kWeightBytes, smem_u32(&bar_w));
        }
    } else if (warp >= kConverterWarp0) {
        // ------------------------------ converters ------------------------------
        // A thread owns up to kItemsPerThread 4-pixel items of a strip (item k = index tid + 128 k, the same row / column
        // for every strip) and a private 16-byte staging slot per item and channel. Its cp.async copies run one strip
        // ahead: as soon as item k of the current strip has been read out of its slots, the copies of item k of the NEXT
        // strip are issued into them (one commit group per item). Before reading item k the thread therefore only
        // has to wait for its OLDEST group (wait_group kItemsPerThread - 1), issued a whole strip earlier, so the
        // global-memory latency never shows; one strip of loads (62 KB) is in flight per SM at all times.
        const int tid = threadIdx.x - kConverterWarp0 * 32;
        const float* x = static_cast<const float*>(p.aux_in);
        const int wq = W >> 2;  // 4-pixel items per row
        const bool vec = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
        const uint32_t my_slot = staging_smem + (uint32_t)tid * 16u;
        uint32_t item_rq[kItemsPerThread];  // row << 16 | 4-pixel column of item k
#pragma unroll
        for (int k = 0; k < kItemsPerThread; ++k) {
            const int idx = tid + k * kConverterThreads;
            const int row = idx / wq;
            item_rq[k] = ((uint32_t)row << 16) | (uint32_t)(idx - row * wq);
        }
        const size_t plane = (size_t)H * W;
        auto strip_geom = [&](int strip, const float** base, int* row_lo, int* row_hi) {
            // rows [row_lo, row_hi) of the strip's local packed rows come from the image plane at `base` (+ local row * W);
            // the others are padding rows (zeros)
            const int n = strip / strips_per_image;
            const int s = strip - n * strips_per_image;
            const int row0 = s > 0 ? 16 * s - 2 : 0;
            int rows_in = (s > 0 ? 2 * (kConvRows - 1) : 2 * (kConvRows - 2)) + kKH;
            if (row0 + rows_in > Hp) rows_in = Hp - row0;
            const int h0 = row0 - p.pad_h;  // image row of local row 0
            *row_lo = h0 < 0 ? -h0 : 0;
            *row_hi = (H - h0) < rows_in ? (H - h0) : rows_in;
            *base = x + (size_t)n * C * plane + (ptrdiff_t)h0 * W;
            return rows_in;
        };
        auto issue_item = [&](int k, const float* base, int row_lo, int row_hi) {  // one commit group, possibly empty
            const int row = (int)(item_rq[k] >> 16), q = (int)(item_rq[k] & 0xffffu);
            if (row >= row_lo && row < row_hi) {
                const float* src = base + (size_t)row * W + 4 * q;
                const uint32_t dst = my_slot + (uint32_t)(k * kMaxC * kConverterThreads) * 16u;
                for (int c = 0; c < C; ++c) {
                    if (vec) {
                        cp_async_16(dst + (uint32_t)(c * kConverterThreads) * 16u, src + c * plane);
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e) cp_async_4(dst + (uint32_t)(c * kConverterThreads) * 16u + 4u * e, src + c * plane + e);
                    }
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        pdl_wait();
        int stage = 0;
        uint32_t phase = 0;
        {
            const float* base = x;
            int row_lo = 0, row_hi = 0;
            if ((int)blockIdx.x < total_strips) strip_geom(blockIdx.x, &base, &row_lo, &row_hi);
#pragma unroll
            for (int k = 0; k < kItemsPerThread; ++k) issue_item(k, base, row_lo, row_hi);
        }
        for (int strip = blockIdx.x; strip < total_strips; strip += gridDim.x) {
            const float* base;
            int row_lo, row_hi;
            const int rows_in = strip_geom(strip, &base, &row_lo, &row_hi);
            const int next = strip + gridDim.x;
            const float* base2 = x;
            int row_lo2 = 0, row_hi2 = 0;  // no next strip: empty groups keep the group count in step
            if (next < total_strips) strip_geom(next, &base2, &row_lo2, &row_hi2);
            // warp-uniform outcome: no lane may leave while the others go on to the __syncwarp below
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&bar_empty[stage]), phase ^ 1u, abort_ptr))) break;
            const uint32_t dst0 = strip_smem + (uint32_t)stage * kStripBytes + (uint32_t)p.pad_w * 8u;
#pragma unroll
            for (int k = 0; k < kItemsPerThread; ++k) {
                const int row = (int)(item_rq[k] >> 16), q = (int)(item_rq[k] & 0xffffu);
                asm volatile("cp.async.wait_group %0;" ::"n"(kItemsPerThread - 1) : "memory");  // this item's copies have landed
                if (row < rows_in) {
                    float4 v[kMaxC];
#pragma unroll
                    for (int c = 0; c < kMaxC; ++c) v[c] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    if (row >= row_lo && row < row_hi) {
#pragma unroll
                        for (int c = 0; c < kMaxC; ++c)
                            if (c < C) {
                                const uint32_t src = my_slot + (uint32_t)((k * kMaxC + c) * kConverterThreads) * 16u;
                                asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v[c].x), "=f"(v[c].y), "=f"(v[c].z), "=f"(v[c].w) : "r"(src));
                            }
                    }
                    const uint32_t dst = dst0 + (uint32_t)row * (uint32_t)row_bytes + (uint32_t)q * 32u;
                    const float* f0 = reinterpret_cast<const float*>(&v[0]);
                    const float* f1 = reinterpret_cast<const float*>(&v[1]);
                    const float* f2 = reinterpret_cast<const float*>(&v[2]);
#pragma unroll
                    for (int px = 0; px < 4; ++px)
                        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(dst + px * 8u), "r"(pack_bf16(f0[px], f1[px])),
                                     "r"(pack_bf16(f2[px], 0.0f))
                                     : "memory");
                }
                // the slots of item k are in registers (their values went into the stores above): refill them
                issue_item(k, base2, row_lo2, row_hi2);
            }
            fence_proxy_async_shared();  // the tensor core reads these bytes through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_full[stage]));
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        cp_async_wait_all();
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        // The whole warp walks the loop (uniform control flow); one elected lane issues the instructions.
        {
            bool ok = __all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&bar_w), 0, abort_ptr));
            const uint32_t ab_hi = desc_hi(128, 0);  // unswizzled, 8-row groups 128 B apart (A and B alike)
            const uint32_t w_lo = (w_smem & 0x3ffffu) >> 4;
            const uint32_t row16 = (uint32_t)(row_bytes >> 4);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t blk = 0;
            for (int strip = blockIdx.x; ok && strip < total_strips; strip += gridDim.x) {
                const int s = strip % strips_per_image;
                if (!__all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&bar_full[stage]), phase, abort_ptr))) break;
                tc_fence_after_sync();
                const uint32_t strip_base = strip_smem + (uint32_t)stage * kStripBytes;
                for (int j0 = (s > 0 ? 0 : 1); j0 < kConvRows; j0 += kBlockRows, ++blk) {
                    const int R = kConvRows - j0 < kBlockRows ? kConvRows - j0 : kBlockRows;
                    const uint32_t buf = blk & 1u;
                    if (!__all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&bar_acc_empty[buf]), ((blk >> 1) & 1u) ^ 1u, abort_ptr))) { ok = false; break; }
                    tc_fence_after_sync();
                    const int in_row0 = s > 0 ? 2 * j0 : 2 * j0 - 2;  // local packed row of filter row 0 of conv row j0
                    const uint32_t a_lo0 = desc_lo(strip_base + (uint32_t)(in_row0 * row_bytes), 16);
                    const uint32_t d0 = tmem_base + buf * kBufCols;
                    if (elect_one()) {
                        if (R == 3) issue_block<3>(d0, a_lo0, row16, ab_hi, w_lo);
                        else if (R == 2) issue_block<2>(d0, a_lo0, row16, ab_hi, w_lo);
                        else issue_block<1>(d0, a_lo0, row16, ab_hi, w_lo);
                        umma_commit(smem_u32(&bar_acc_full[buf]));
                    }
                    __syncwarp();
                }
                if (!ok) break;
                if (elect_one()) umma_commit(smem_u32(&bar_empty[stage]));
                __syncwarp();
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
        }
    } else {
        // ------------------------------ epilogue ------------------------------
        // TMEM lane quadrant (warp & 3) x one channel part of kPartCols channels per warp.
        const int quad = warp & 3;
        const int part = (warp - kEpilogueWarp0) >> 2;
        const int ow = quad * 32 + lane;
        const int c0 = part * kPartCols;
        const int POH = p.OH / 2, POW = p.OW / 2;
        __nv_bfloat16* pooled = static_cast<__nv_bfloat16*>(p.out);
        const bool col_ok = ow < p.OW;
        constexpr int kPairs = kPartCols / 2;  // packed bf16 pairs a thread holds
        float bias[kPartCols];
#pragma unroll
        for (int e = 0; e < kPartCols; ++e) bias[e] = p.bias != nullptr ? __ldg(p.bias + c0 + e) : 0.0f;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0;
        pdl_wait();
        uint32_t blk = 0;
        uint32_t fin = 0;  // pooled rows finished so far (parity picks the exchange slot)
        bool bad = false, dead = false;
        for (int strip = blockIdx.x; !dead && strip < total_strips; strip += gridDim.x) {
            const int n = strip / strips_per_image;
            const int s = strip - n * strips_per_image;
            uint32_t vmax[kPairs];  // running maximum over the conv rows of the current pooled row (0 is neutral)
#pragma unroll
            for (int e = 0; e < kPairs; ++e) vmax[e] = 0u;
            for (int j0 = (s > 0 ? 0 : 1); !dead && j0 < kConvRows; j0 += kBlockRows, ++blk) {
                const int R = kConvRows - j0 < kBlockRows ? kConvRows - j0 : kBlockRows;
                const uint32_t buf = blk & 1u;
                // A wait that runs out is carried to the next 128-thread barrier, where the four warps of this channel
                // part learn of it and leave together.
                if (!bad) bad = !__all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&bar_acc_full[buf]), (blk >> 1) & 1u, abort_ptr));
                if (!bad) tc_fence_after_sync();
                for (int jj = 0; jj < R; ++jj) {
                    const int j = j0 + jj;
                    uint32_t pk[kPairs];
#pragma unroll
                    for (int e = 0; e < kPairs; ++e) pk[e] = 0u;
                    if (!bad) {
                        uint32_t v[kPartCols];
                        tmem_ld_part(lane_base + buf * kBufCols + (uint32_t)(jj * kBN), v);
                        tmem_ld_wait();
                        if (jj == R - 1) {  // the buffer is in registers: hand it back before the arithmetic
                            tc_fence_before_sync();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[buf]));
                        }
                        if (col_ok) {  // columns beyond the image (the M = 128 tile is wider) stay neutral
#pragma unroll
                            for (int e = 0; e < kPairs; ++e)
                                pk[e] = pack_bf16(__fadd_rn(__uint_as_float(v[2 * e]), bias[2 * e]),
                                                  __fadd_rn(__uint_as_float(v[2 * e + 1]), bias[2 * e + 1]));
                        }
                    }
#pragma unroll
                    for (int e = 0; e < kPairs; ++e) {
                        const __nv_bfloat162 m = __hmax2(*reinterpret_cast<__nv_bfloat162*>(&vmax[e]), *reinterpret_cast<__nv_bfloat162*>(&pk[e]));
                        vmax[e] = *reinterpret_cast<const uint32_t*>(&m);
                    }
                    // local rows 2, 4, 6, 8 close a pooled row (and open the next one)
                    if ((j & 1) == 0 && j >= 2) {
                        if (lane == 31) {  // the left neighbour of the next quadrant's first column
                            const uint32_t slot = exch_smem + ((((fin & 1u) * (uint32_t)(64 / kPartCols) + (uint32_t)part) * 4u + (uint32_t)quad) * (uint32_t)(kPartCols * 2));
#pragma unroll
                            for (int g = 0; g < kPairs / 4; ++g)
                                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(slot + g * 16u), "r"(vmax[4 * g]), "r"(vmax[4 * g + 1]),
                                             "r"(vmax[4 * g + 2]), "r"(vmax[4 * g + 3])
                                             : "memory");
                        }
                        if (named_barrier_or(1 + part, 128, bad)) {
                            dead = true;
                            break;
                        }
                        // Horizontal maximum over conv columns 2m-1, 2m, 2m+1 for pooled column m, shared by the two lanes
                        // of a pair: the even lane (column 2m) takes the lower half of the part's channels, the odd lane
                        // (column 2m+1) the upper half, so each register costs three shuffles per PAIR of lanes instead
                        // of four and every lane stores.
                        constexpr int kHalf = kPairs / 2;
                        const bool odd = (lane & 1) != 0;
                        uint32_t edge[kHalf];  // column 2m-1 for lanes 0 and 1: the previous quadrant's last column (or padding)
#pragma unroll
                        for (int e = 0; e < kHalf; ++e) edge[e] = 0u;
                        if (lane < 2 && quad > 0) {
                            const uint32_t slot = exch_smem + ((((fin & 1u) * (uint32_t)(64 / kPartCols) + (uint32_t)part) * 4u + (uint32_t)(quad - 1)) * (uint32_t)(kPartCols * 2)) +
                                                  (odd ? (uint32_t)(kHalf * 4) : 0u);
#pragma unroll
                            for (int g = 0; g < kHalf / 4; ++g)
                                asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                             : "=r"(edge[4 * g]), "=r"(edge[4 * g + 1]), "=r"(edge[4 * g + 2]), "=r"(edge[4 * g + 3])
                                             : "r"(slot + g * 16u));
                        }
                        const __nv_bfloat162 zero2 = __floats2bfloat162_rn(0.0f, 0.0f);
                        uint32_t res[kHalf];
#pragma unroll
                        for (int e = 0; e < kHalf; ++e) {
                            const uint32_t lo = vmax[e], hi = vmax[e + kHalf];
                            const uint32_t mine = odd ? hi : lo;
                            const uint32_t partner = __shfl_xor_sync(0xffffffffu, odd ? lo : hi, 1);  // the pair's other column, my half
                            const uint32_t up1 = __shfl_up_sync(0xffffffffu, lo, 1);                    // even lanes: column 2m-1, lower half
                            const uint32_t up2 = __shfl_up_sync(0xffffffffu, hi, 2);                    // odd lanes: column 2m-1, upper half
                            uint32_t prev = odd ? up2 : up1;
                            if (lane < 2) prev = edge[e];
                            __nv_bfloat162 m = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&mine), *reinterpret_cast<const __nv_bfloat162*>(&partner));
                            m = __hmax2(m, *reinterpret_cast<const __nv_bfloat162*>(&prev));
                            m = __hmax2(m, zero2);  // ReLU
                            res[e] = *reinterpret_cast<uint32_t*>(&m);
                        }
                        if ((ow & ~1) < p.OW) {
                            const int ph = 4 * s + j / 2 - 1;
                            uint4* dst = reinterpret_cast<uint4*>(pooled + ((((size_t)n * POH + ph) * POW + (ow >> 1)) * kBN) + c0 + (odd ? kHalf * 2 : 0));
#pragma unroll
                            for (int g = 0; g < kHalf / 4; ++g) dst[g] = make_uint4(res[4 * g], res[4 * g + 1], res[4 * g + 2], res[4 * g + 3]);
                        }
                        ++fin;
#pragma unroll
                        for (int e = 0; e < kPairs; ++e) vmax[e] = pk[e];  // the running maximum restarts with this row
                    }
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

// Stem weights, filter rows stacked by parity: [r = 6,4,2,0 | r = 5,3,1], each stack in core-matrix order
// [4 k-chunks][stack rows][8] bf16 with stack row = (position in the stack) * 64 + cout; element e of chunk j = pixel
// 2j + e/4, channel e%4; zero for kw >= KW or c >= C.
__global__ void stem_pack_weights_stacked_kernel(const float* __restrict__ w, __nv_bfloat16* __restrict__ out, int O, int C, int KW) {
    const int total = 4 * (kEvenRows + kOddRows) * 8;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const bool odd = i >= 4 * kEvenRows * 8;
        const int li = odd ? i - 4 * kEvenRows * 8 : i;
        const int rows = odd ? kOddRows : kEvenRows;
        const int e = li & 7;
        const int row = (li >> 3) % rows;
        const int jc = (li >> 3) / rows;
        const int o = row & (kBN - 1), pos = row / kBN;
        const int r = odd ? (kKH - 2) - 2 * pos : (kKH - 1) - 2 * pos;
        const int kw = 2 * jc + (e >> 2), c = e & 3;
        float f = 0.0f;
        if (o < O && c < C && kw < KW) f = w[((o * C + c) * kKH + r) * KW + kw];
        out[i] = __float2bfloat16_rn(f);
    }
}

}  // namespace

bool stem_pool_nchw_applicable(TcDType dtype, int C, int O, int KH, int KW, int W, int OH, int OW, int Wp) {
    return dtype == kTcBF16 && C >= 1 && C <= kMaxC && W <= 4 * kMaxRowItems && kInRows * (W / 4) <= kItemsPerThread * kConverterThreads &&
           O == kBN && KH == kKH && KW <= 8 && (W % 4) == 0 && (OH % (2 * kPooledRows)) == 0 &&
           (OW % 2) == 0 && OW <= 128 && Wp * 8 <= kMaxRowBytes && (Wp * 8) % 16 == 0;
}

size_t stem_stacked_weight_bytes() { return (size_t)kWeightBytes; }

int32_t stem_stacked_pack_weights(const float* w, void* out, int O, int C, int KW, cudaStream_t s) {
    stem_pack_weights_stacked_kernel<<<(4 * (kEvenRows + kOddRows) * 8 + 255) / 256, 256, 0, s>>>(w, static_cast<__nv_bfloat16*>(out), O, C, KW);
    return check_launch("stem_pack_weights_stacked");
}

int32_t stem_pool_nchw_setup(TcParams* p, const void* packed_w, int N, int C, int H, int W, int OH, int OW, int pad_h, int pad_w,
                             int Hp, int Wp) {
    p->N = N; p->OH = OH; p->OW = OW; p->Cout = kBN;
    p->taps_h = kKH; p->taps_w = 1; p->stride = 2;
    p->pad_h = pad_h; p->pad_w = pad_w; p->dil_h = 1; p->dil_w = 1;
    p->BW = 128; p->BH = kBlockRows; p->BNI = 1;
    p->tiles_w = 1; p->tiles_h = OH; p->tiles_n = N; p->tiles_c = 1;
    p->aux_in = nullptr;  // the graph input: bound at run time
    p->aux_w = packed_w;
    p->aux_row_bytes = Wp * 8;
    p->aux_hp = Hp;
    p->aux_c = C; p->aux_h = H; p->aux_w_px = W;
    KXC_TRY(tc_status_word(&p->status));
    return KXC_B200_OK;
}

int32_t stem_pool_nchw_launch(const TcParams& p, cudaStream_t stream) {
    static PerDeviceOnce smem_once;
    KXC_TRY(smem_opt_in(smem_once, conv_stem_pool_nchw_kernel, kSmemBytes));
    if (!p.vec_ok || p.out == nullptr || p.aux_in == nullptr)
        return fail(KXC_B200_ERR_INVALID, "fused stem conv + pool: missing tensors or pointers that are not 16-byte aligned");
    if (!p.relu) return fail(KXC_B200_ERR_INVALID, "fused stem conv + pool: the pooling shortcut relies on the ReLU in between");
    const long long strips = (long long)(p.OH / (2 * kPooledRows)) * p.N;
    if (strips <= 0) return KXC_B200_OK;
    const int grid = (int)(strips < kNumSMs ? strips : kNumSMs);
    KXC_CUDA_TRY(launch_kernel(conv_stem_pool_nchw_kernel, dim3(grid), dim3(kThreads), kSmemBytes, stream, /*pdl=*/true, 1, p));
    return check_launch("conv_stem_pool_nchw_kernel");
}

}  // namespace kxc_b200

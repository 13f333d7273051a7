// transpose, reshape and cast on tensors in the reference's dense row-major layout. All three only move or convert
// elements, so they are bound by HBM bandwidth and bit-exact.
//
//   transpose  out[i0..] = in[...] with in_index[perm[k]] = out_index[k] (include/te/topi/transform.h:20-52 via
//              TransposeCompute, src/relay/op/tensor/transform.cc:206-212). Dimensions that stay adjacent are merged
//              first. When the input's fastest dimension is not the output's, 32x32 tiles go through shared memory so
//              that both the reads and the writes are coalesced; otherwise rows are copied as they are.
//   reshape    out[flat] = in[flat] (ReshapeCompute, transform.cc:185-204): a copy.
//   cast       one conversion per element with the semantics of CodeGenLLVM::CastValue (src/codegen/codegen_llvm.cc:219-248):
//              integer widening by the SOURCE's signedness, truncation by dropping high bits, float -> integer toward
//              zero, integer -> float and double -> float to nearest even. A float that does not fit the integer type is
//              undefined in the reference (fptosi / fptoui); here it saturates and NaN gives 0.
#include <type_traits>

#include "common.cuh"

namespace kxc_b200 {
namespace {

constexpr int kTile = 32;
constexpr int kTileRows = 8;  // 32 x 8 threads, 4 rows each

struct TransposeDims {
    int rank;              // merged output rank
    int64_t shape[6];      // merged output extents
    int64_t istride[6];    // input stride (in elements) of each output dimension
    int64_t total;
};

// General form: consecutive threads take consecutive output elements. Coalesced on both sides when the last output
// dimension is also contiguous in the input (istride == 1). Index arithmetic is 32-bit when the tensor allows it
// (64-bit divisions cost more than the copy); two elements are in flight per thread.
template <typename I>
__device__ __forceinline__ int64_t transpose_src_offset(I o, const TransposeDims& d) {
    I rem = o;
    int64_t off = 0;
#pragma unroll
    for (int j = 5; j >= 0; --j) {
        if (j < d.rank) {
            const I ext = (I)d.shape[j];
            const I q = rem / ext;
            off += (int64_t)(rem - q * ext) * d.istride[j];
            rem = q;
        }
    }
    return off;
}

template <typename T, typename I>
__global__ void __launch_bounds__(256) transpose_rows_kernel(const T* __restrict__ in, T* __restrict__ out, TransposeDims d) {
    const I total = (I)d.total, stride = (I)gridDim.x * 256;
    I o = (I)blockIdx.x * 256 + threadIdx.x;
    for (; o + stride < total; o += 2 * stride) {
        const T a = __ldg(in + transpose_src_offset<I>(o, d));
        const T b = __ldg(in + transpose_src_offset<I>(o + stride, d));
        out[o] = a;
        out[o + stride] = b;
    }
    if (o < total) out[o] = __ldg(in + transpose_src_offset<I>(o, d));
}

struct TileDims {
    int64_t X, Y;            // X: extent of the output's fastest dimension; Y: extent of the input's fastest dimension
    int64_t x_istride;       // input stride of X (Y's input stride is 1)
    int64_t y_ostride;       // output stride of Y (X's output stride is 1)
    int nb;                  // remaining ("batch") dimensions
    int64_t bshape[4], b_istride[4], b_ostride[4];
    int64_t tiles_x, tiles_y, tiles;
};

template <typename T>
__global__ void __launch_bounds__(kTile* kTileRows) transpose_tiles_kernel(const T* __restrict__ in, T* __restrict__ out, TileDims d) {
    __shared__ T tile[kTile][kTile + 1];
    const int tx = threadIdx.x & (kTile - 1), ty = threadIdx.x / kTile;
    for (int64_t t = blockIdx.x; t < d.tiles; t += gridDim.x) {
        int64_t rem = t;
        const int64_t bx = rem % d.tiles_x;
        rem /= d.tiles_x;
        const int64_t by = rem % d.tiles_y;
        rem /= d.tiles_y;
        int64_t ibase = 0, obase = 0;
#pragma unroll
        for (int j = 3; j >= 0; --j) {
            if (j < d.nb) {
                const int64_t q = rem / d.bshape[j];
                const int64_t i = rem - q * d.bshape[j];
                ibase += i * d.b_istride[j];
                obase += i * d.b_ostride[j];
                rem = q;
            }
        }
        const int64_t x0 = bx * kTile, y0 = by * kTile;
        // read: threadIdx.x runs along Y (contiguous in the input)
        T v[kTile / kTileRows];
#pragma unroll
        for (int k = 0; k < kTile / kTileRows; ++k) {  // all loads are issued before the first shared-memory store
            const int64_t x = x0 + ty + k * kTileRows, y = y0 + tx;
            v[k] = (x < d.X && y < d.Y) ? __ldg(in + ibase + x * d.x_istride + y) : T{};
        }
#pragma unroll
        for (int k = 0; k < kTile / kTileRows; ++k) tile[ty + k * kTileRows][tx] = v[k];
        __syncthreads();
        // write: threadIdx.x runs along X (contiguous in the output)
#pragma unroll
        for (int r = ty; r < kTile; r += kTileRows) {
            const int64_t y = y0 + r, x = x0 + tx;
            if (x < d.X && y < d.Y) out[obase + y * d.y_ostride + x] = tile[tx][r];
        }
        __syncthreads();
    }
}

// 4-byte elements with 16-byte accesses on both sides: a 64x64 tile, 256 threads. Each thread reads float4s along Y
// (16 threads cover one 256-byte row of the tile), the tile sits transposed in shared memory, and each thread writes
// float4s along X. Needs X, Y, the two strides and the batch strides to be multiples of 4 elements and 16-byte aligned
// pointers; tiles at the ragged edges are clipped per float4 (X and Y being multiples of 4 keeps every float4 whole).
constexpr int kVTile = 64;

__global__ void __launch_bounds__(256) transpose_tiles_vec4_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out,
                                                                  TileDims d) {
    __shared__ uint32_t tile[kVTile][kVTile + 1];  // tile[x][y]
    const int lane16 = threadIdx.x & 15, row16 = threadIdx.x >> 4;  // 16 float4 per 64-element row, 16 rows per pass
    for (int64_t t = blockIdx.x; t < d.tiles; t += gridDim.x) {
        int64_t rem = t;
        const int64_t bx = rem % d.tiles_x;
        rem /= d.tiles_x;
        const int64_t by = rem % d.tiles_y;
        rem /= d.tiles_y;
        int64_t ibase = 0, obase = 0;
#pragma unroll
        for (int j = 3; j >= 0; --j) {
            if (j < d.nb) {
                const int64_t q = rem / d.bshape[j];
                const int64_t i = rem - q * d.bshape[j];
                ibase += i * d.b_istride[j];
                obase += i * d.b_ostride[j];
                rem = q;
            }
        }
        const int64_t x0 = bx * kVTile, y0 = by * kVTile;
        uint4 v[kVTile / 16];
#pragma unroll
        for (int k = 0; k < kVTile / 16; ++k) {  // input rows x, float4 along y
            const int64_t x = x0 + row16 + k * 16, y = y0 + lane16 * 4;
            v[k] = (x < d.X && y < d.Y) ? __ldg(reinterpret_cast<const uint4*>(in + ibase + x * d.x_istride + y)) : uint4{0, 0, 0, 0};
        }
#pragma unroll
        for (int k = 0; k < kVTile / 16; ++k) {
            const int x = row16 + k * 16, y = lane16 * 4;
            tile[x][y] = v[k].x;
            tile[x][y + 1] = v[k].y;
            tile[x][y + 2] = v[k].z;
            tile[x][y + 3] = v[k].w;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kVTile / 16; ++k) {  // output rows y, float4 along x
            const int yl = row16 + k * 16, xl = lane16 * 4;
            const int64_t y = y0 + yl, x = x0 + xl;
            if (x < d.X && y < d.Y) {
                const uint4 w{tile[xl][yl], tile[xl + 1][yl], tile[xl + 2][yl], tile[xl + 3][yl]};
                *reinterpret_cast<uint4*>(out + obase + y * d.y_ostride + x) = w;
            }
        }
        __syncthreads();
    }
}

int grid_for(int64_t blocks) {
    const int64_t cap = (int64_t)kNumSMs * 16;
    return (int)(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

template <typename T>
int32_t rows_launch(const void* in, void* out, const TransposeDims& m, cudaStream_t s) {
    const int grid = grid_for((m.total + 511) / 512);
    if (m.total < (int64_t)1 << 31)
        transpose_rows_kernel<T, uint32_t><<<grid, 256, 0, s>>>(static_cast<const T*>(in), static_cast<T*>(out), m);
    else
        transpose_rows_kernel<T, int64_t><<<grid, 256, 0, s>>>(static_cast<const T*>(in), static_cast<T*>(out), m);
    return check_launch("transpose");
}

template <typename T>
int32_t transpose_launch(const void* in, void* out, const TransposeDims& m, const int64_t* ostride, cudaStream_t s) {
    const int last = m.rank - 1;
    if (m.istride[last] == 1) return rows_launch<T>(in, out, m, s);
    int q = -1;  // the output dimension that is contiguous in the input
    for (int j = 0; j < m.rank; ++j)
        if (m.istride[j] == 1) q = j;
    if (q < 0 || m.rank - 2 > 4) return rows_launch<T>(in, out, m, s);  // cannot happen for at most 6 merged dimensions
    TileDims d{};
    d.X = m.shape[last];
    d.Y = m.shape[q];
    d.x_istride = m.istride[last];
    d.y_ostride = ostride[q];
    for (int j = 0; j < m.rank; ++j) {
        if (j == q || j == last) continue;
        d.bshape[d.nb] = m.shape[j];
        d.b_istride[d.nb] = m.istride[j];
        d.b_ostride[d.nb] = ostride[j];
        ++d.nb;
    }
    if (sizeof(T) == 4 && aligned16(in) && aligned16(out)) {
        bool vec = d.X % 4 == 0 && d.Y % 4 == 0 && d.x_istride % 4 == 0 && d.y_ostride % 4 == 0;
        for (int j = 0; j < d.nb; ++j) vec = vec && d.b_istride[j] % 4 == 0 && d.b_ostride[j] % 4 == 0;
        if (vec) {
            d.tiles_x = (d.X + kVTile - 1) / kVTile;
            d.tiles_y = (d.Y + kVTile - 1) / kVTile;
            d.tiles = d.tiles_x * d.tiles_y;
            for (int j = 0; j < d.nb; ++j) d.tiles *= d.bshape[j];
            transpose_tiles_vec4_kernel<<<grid_for(d.tiles), 256, 0, s>>>(static_cast<const uint32_t*>(in), static_cast<uint32_t*>(out), d);
            return check_launch("transpose");
        }
    }
    d.tiles_x = (d.X + kTile - 1) / kTile;
    d.tiles_y = (d.Y + kTile - 1) / kTile;
    d.tiles = d.tiles_x * d.tiles_y;
    for (int j = 0; j < d.nb; ++j) d.tiles *= d.bshape[j];
    transpose_tiles_kernel<T><<<grid_for(d.tiles), kTile * kTileRows, 0, s>>>(static_cast<const T*>(in), static_cast<T*>(out), d);
    return check_launch("transpose");
}

// One element. Integer sources and float -> float are the language's conversions (they are what sext/zext/trunc,
// sitofp/uitofp and fpext/fptrunc do); float -> integer goes toward zero and saturates at the type's limits.
template <typename S, typename D>
__device__ __forceinline__ D convert_elem(S v) {
    if constexpr ((std::is_same<S, float>::value || std::is_same<S, double>::value) && std::is_integral<D>::value) {
        if constexpr (sizeof(D) == 8) {
            if constexpr (std::is_same<S, float>::value) return (D)__float2ll_rz(v);
            else return (D)__double2ll_rz(v);
        } else {
            int r;
            if constexpr (std::is_same<S, float>::value) r = __float2int_rz(v);
            else r = __double2int_rz(v);
            if constexpr (sizeof(D) == 1) {
                const int lo = std::is_signed<D>::value ? -128 : 0, hi = std::is_signed<D>::value ? 127 : 255;
                r = r < lo ? lo : (r > hi ? hi : r);
            }
            return (D)r;
        }
    } else {
        return static_cast<D>(v);
    }
}

template <typename S, typename D>
__global__ void __launch_bounds__(256) cast_kernel(const S* __restrict__ in, D* __restrict__ out, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < n; i += 4 * stride) {  // four independent loads in flight per thread
        const S a = __ldg(in + i), b = __ldg(in + i + stride), c = __ldg(in + i + 2 * stride), e = __ldg(in + i + 3 * stride);
        out[i] = convert_elem<S, D>(a);
        out[i + stride] = convert_elem<S, D>(b);
        out[i + 2 * stride] = convert_elem<S, D>(c);
        out[i + 3 * stride] = convert_elem<S, D>(e);
    }
    for (; i < n; i += stride) out[i] = convert_elem<S, D>(__ldg(in + i));
}

// V consecutive elements per thread, moved as aligned vectors (the wider of the two types takes 32 bytes per thread).
template <typename T, int V>
struct alignas(sizeof(T) * V) ElemVec {
    T v[V];
};

template <typename S, typename D, int V>
__global__ void __launch_bounds__(256) cast_vec_kernel(const S* __restrict__ in, D* __restrict__ out, int64_t n) {
    const int64_t nv = n / V;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const ElemVec<S, V>* in_v = reinterpret_cast<const ElemVec<S, V>*>(in);
    ElemVec<D, V>* out_v = reinterpret_cast<ElemVec<D, V>*>(out);
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + stride < nv; i += 2 * stride) {
        const ElemVec<S, V> a = in_v[i], b = in_v[i + stride];
        ElemVec<D, V> ra, rb;
#pragma unroll
        for (int k = 0; k < V; ++k) {
            ra.v[k] = convert_elem<S, D>(a.v[k]);
            rb.v[k] = convert_elem<S, D>(b.v[k]);
        }
        out_v[i] = ra;
        out_v[i + stride] = rb;
    }
    if (i < nv) {
        const ElemVec<S, V> a = in_v[i];
        ElemVec<D, V> ra;
#pragma unroll
        for (int k = 0; k < V; ++k) ra.v[k] = convert_elem<S, D>(a.v[k]);
        out_v[i] = ra;
    }
    // the last n % V elements
    const int64_t t = nv * V + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n) out[t] = convert_elem<S, D>(in[t]);
}

template <typename S, typename D>
int32_t cast_launch(const void* in, void* out, int64_t n, cudaStream_t s) {
    constexpr int kWide = sizeof(S) > sizeof(D) ? sizeof(S) : sizeof(D);
    constexpr int V = 32 / kWide;  // 4 (8-byte types), 8 (4-byte) or 32 (1-byte)
    const bool aligned = (reinterpret_cast<uintptr_t>(in) % (sizeof(S) * V) == 0) && (reinterpret_cast<uintptr_t>(out) % (sizeof(D) * V) == 0);
    if (aligned && n >= V) {
        const int64_t nv = n / V;
        cast_vec_kernel<S, D, V><<<grid_for((nv + 511) / 512), 256, 0, s>>>(static_cast<const S*>(in), static_cast<D*>(out), n);
    } else {
        cast_kernel<S, D><<<grid_for((n + 1023) / 1024), 256, 0, s>>>(static_cast<const S*>(in), static_cast<D*>(out), n);
    }
    return check_launch("cast");
}

template <typename S>
int32_t cast_from(const void* in, void* out, int32_t to, int64_t n, cudaStream_t s) {
    switch (to) {
        case KXC_B200_DT_F32: return cast_launch<S, float>(in, out, n, s);
        case KXC_B200_DT_I32: return cast_launch<S, int32_t>(in, out, n, s);
        case KXC_B200_DT_I64: return cast_launch<S, int64_t>(in, out, n, s);
        case KXC_B200_DT_F64: return cast_launch<S, double>(in, out, n, s);
        case KXC_B200_DT_I8: return cast_launch<S, int8_t>(in, out, n, s);
        case KXC_B200_DT_U8: return cast_launch<S, uint8_t>(in, out, n, s);
        default: return fail(KXC_B200_ERR_UNSUPPORTED, "cast: target dtype code %d is not supported", to);
    }
}

int dtype_bytes(int32_t code) {
    switch (code) {
        case KXC_B200_DT_F32: case KXC_B200_DT_I32: return 4;
        case KXC_B200_DT_I64: case KXC_B200_DT_F64: return 8;
        case KXC_B200_DT_I8: case KXC_B200_DT_U8: return 1;
        default: return 0;
    }
}

}  // namespace
}  // namespace kxc_b200

using namespace kxc_b200;

extern "C" int32_t kxc_b200_transpose(void** packed_args, const kxc_b200_transpose_desc* desc, void* stream) {
    KXC_TRY(require_device());
    if (!packed_args || !desc) return fail(KXC_B200_ERR_INVALID, "transpose: bad arguments");
    const int rank = desc->rank;
    if (rank < 1 || rank > 6) return fail(KXC_B200_ERR_INVALID, "transpose: rank must be in [1,6]");
    if (desc->elem_bytes != 4 && desc->elem_bytes != 8 && desc->elem_bytes != 1)
        return fail(KXC_B200_ERR_INVALID, "transpose: elem_bytes must be 1, 4 or 8");
    int perm[6];
    bool seen[6] = {false, false, false, false, false, false};
    for (int i = 0; i < rank; ++i) {
        int a = desc->num_axes == 0 ? rank - 1 - i : desc->perm[i];  // no axes: reverse the dimensions
        if (desc->num_axes != 0 && desc->num_axes != rank) return fail(KXC_B200_ERR_INVALID, "transpose perm rank mismatch");
        if (a < 0) a += rank;
        if (a < 0 || a >= rank) return fail(KXC_B200_ERR_INVALID, "transpose: axis %d out of range", desc->perm[i]);
        if (seen[a]) return fail(KXC_B200_ERR_INVALID, "transpose duplicate axis");
        seen[a] = true;
        perm[i] = a;
    }
    int64_t istr[6], st = 1, total = 1;
    for (int i = rank - 1; i >= 0; --i) {
        if (desc->shape[i] < 0) return fail(KXC_B200_ERR_INVALID, "transpose: negative extent");
        istr[i] = st;
        st *= desc->shape[i];
        total *= desc->shape[i];
    }
    if (total == 0) return KXC_B200_OK;
    if (!packed_args[0] || !packed_args[1]) return fail(KXC_B200_ERR_INVALID, "transpose: null tensor pointer");
    // merge output dimensions that are neighbours in the input too; drop extent-1 dimensions
    TransposeDims m{};
    for (int i = 0; i < rank; ++i) {
        const int64_t ext = desc->shape[perm[i]], is = istr[perm[i]];
        if (ext == 1) continue;
        if (m.rank > 0 && m.istride[m.rank - 1] == is * ext) {
            m.shape[m.rank - 1] *= ext;
            m.istride[m.rank - 1] = is;
        } else {
            m.shape[m.rank] = ext;
            m.istride[m.rank] = is;
            ++m.rank;
        }
    }
    m.total = total;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (m.rank <= 1) {  // the permutation does not move anything
        if (packed_args[0] != packed_args[1])
            KXC_CUDA_TRY(cudaMemcpyAsync(packed_args[1], packed_args[0], (size_t)total * desc->elem_bytes, cudaMemcpyDeviceToDevice, s));
        return KXC_B200_OK;
    }
    if (packed_args[0] == packed_args[1]) return fail(KXC_B200_ERR_INVALID, "transpose: in-place is not supported");
    int64_t ostr[6];
    st = 1;
    for (int i = m.rank - 1; i >= 0; --i) {
        ostr[i] = st;
        st *= m.shape[i];
    }
    const int last = m.rank - 1;
    if (m.istride[last] == 1 && (m.shape[last] * desc->elem_bytes) % 16 == 0 && aligned16(packed_args[0]) && aligned16(packed_args[1])) {
        // rows are contiguous on both sides and every row starts on a 16-byte boundary (all other strides are multiples
        // of the row length): move 16-byte elements
        const int64_t per = 16 / desc->elem_bytes;
        m.shape[last] /= per;
        m.total /= per;
        for (int i = 0; i < last; ++i) m.istride[i] /= per;
        return rows_launch<uint4>(packed_args[0], packed_args[1], m, s);
    }
    switch (desc->elem_bytes) {
        case 4: return transpose_launch<uint32_t>(packed_args[0], packed_args[1], m, ostr, s);
        case 8: return transpose_launch<uint64_t>(packed_args[0], packed_args[1], m, ostr, s);
        default: return transpose_launch<uint8_t>(packed_args[0], packed_args[1], m, ostr, s);
    }
}

extern "C" int32_t kxc_b200_reshape(void** packed_args, int64_t numel, int32_t elem_bytes, void* stream) {
    KXC_TRY(require_device());
    if (!packed_args || numel < 0 || elem_bytes <= 0) return fail(KXC_B200_ERR_INVALID, "reshape: bad arguments");
    if (numel == 0 || packed_args[0] == packed_args[1]) return KXC_B200_OK;
    if (!packed_args[0] || !packed_args[1]) return fail(KXC_B200_ERR_INVALID, "reshape: null tensor pointer");
    KXC_CUDA_TRY(cudaMemcpyAsync(packed_args[1], packed_args[0], (size_t)numel * (size_t)elem_bytes, cudaMemcpyDeviceToDevice,
                                 static_cast<cudaStream_t>(stream)));
    return KXC_B200_OK;
}

extern "C" int32_t kxc_b200_cast(void** packed_args, int64_t numel, int32_t from, int32_t to, void* stream) {
    KXC_TRY(require_device());
    if (!packed_args || numel < 0) return fail(KXC_B200_ERR_INVALID, "cast: bad arguments");
    if (from == KXC_B200_DT_BOOL || to == KXC_B200_DT_BOOL)
        return fail(KXC_B200_ERR_UNSUPPORTED, "cast: bool is not supported (the reference converts to a 1-bit integer, which keeps only "
                                             "the lowest bit of an integer and is undefined for floats other than 0 and 1)");
    if (!dtype_bytes(from) || !dtype_bytes(to)) return fail(KXC_B200_ERR_INVALID, "cast has unsupported dtype code: %d", dtype_bytes(from) ? to : from);
    if (numel == 0) return KXC_B200_OK;
    if (!packed_args[0] || !packed_args[1]) return fail(KXC_B200_ERR_INVALID, "cast: null tensor pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (from == to) {
        if (packed_args[0] != packed_args[1])
            KXC_CUDA_TRY(cudaMemcpyAsync(packed_args[1], packed_args[0], (size_t)numel * dtype_bytes(from), cudaMemcpyDeviceToDevice, s));
        return KXC_B200_OK;
    }
    switch (from) {
        case KXC_B200_DT_F32: return cast_from<float>(packed_args[0], packed_args[1], to, numel, s);
        case KXC_B200_DT_I32: return cast_from<int32_t>(packed_args[0], packed_args[1], to, numel, s);
        case KXC_B200_DT_I64: return cast_from<int64_t>(packed_args[0], packed_args[1], to, numel, s);
        case KXC_B200_DT_F64: return cast_from<double>(packed_args[0], packed_args[1], to, numel, s);
        case KXC_B200_DT_I8: return cast_from<int8_t>(packed_args[0], packed_args[1], to, numel, s);
        default: return cast_from<uint8_t>(packed_args[0], packed_args[1], to, numel, s);
    }
}

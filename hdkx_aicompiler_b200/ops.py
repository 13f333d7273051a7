"""Operator API on CUDA tensors, one function per Relay op of the reference's ResNet path.

Names, argument meaning and error behaviour follow the reference's operator registry
(src/relay/op/nn/*.cc, src/relay/op/tensor/math.cc): tensors are NCHW / OIHW float32, padding of
nn_conv2d is symmetric (padding[0], padding[1]), pooling padding is (top, left, bottom, right), and a
failing kernel raises `KxcError("Kernel <name> returned error code N")`.

torch is used only to hold device memory and the current stream; all arithmetic happens in
libkxc_b200.so through the C ABI of include/kxc_b200.h.
"""
import torch

from . import _lib
from ._lib import (BIAS, NHWC, PREC_BF16, PREC_FP32, PREC_SIMT, PREC_TF32, RELU, RESIDUAL, AddDesc, Conv2dDesc, GemmDesc,
                   Pool2dDesc, check, load, packed)

PRECISIONS = {"fp32": PREC_FP32, "tf32": PREC_TF32, "bf16": PREC_BF16, "simt": PREC_SIMT, "tf32x3": _lib.PREC_TF32X3}


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _req(t, dtype, name):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ValueError(f"{name}: expected a CUDA tensor (libkxc_b200 has no CPU path)")
    if t.dtype != dtype:
        raise ValueError(f"{name}: expected dtype {dtype}, got {t.dtype}")
    return t.contiguous()


def _pair(v, default):
    v = list(v) if v is not None else []
    return (int(v[0]), int(v[1])) if len(v) >= 2 else (default, default)


def conv_out_dim(n, k, s, p, d=1):
    return (n + 2 * p - ((k - 1) * d + 1)) // s + 1


def pool_out_dim(n, k, s, p0, p1, ceil_mode=False):
    num = n + p0 + p1 - k
    return (num + s - 1) // s + 1 if ceil_mode else num // s + 1


def nn_conv2d(data, weight, bias=None, strides=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1, residual=None,
              relu=False, precision="tf32", out=None):
    """nn_conv2d(data, weight[, bias]) with the optional fused epilogue +residual -> relu.

    `precision`: "fp32" (CUDA cores, reference order, bit-exact), "tf32" or "bf16" (tcgen05 tensor cores)."""
    data = _req(data, torch.float32, "nn_conv2d data")
    weight = _req(weight, torch.float32, "nn_conv2d weight")
    if data.dim() != 4 or weight.dim() != 4:
        raise ValueError("nn_conv2d currently expects NCHW/OIHW rank-4 tensors")
    if groups != 1:
        raise ValueError("nn_conv2d: groups != 1 is not supported")
    N, C, H, W = data.shape
    O, C2, KH, KW = weight.shape
    if C2 != C:
        raise ValueError("nn_conv2d: weight input channels do not match data")
    sh, sw = _pair(strides, 1)
    ph, pw = _pair(padding, 0)
    dh, dw = _pair(dilation, 1)
    OH, OW = conv_out_dim(H, KH, sh, ph, dh), conv_out_dim(W, KW, sw, pw, dw)
    flags = 0
    ptrs = [data.data_ptr(), weight.data_ptr()]
    keep = [data, weight]
    if bias is not None:
        bias = _req(bias, torch.float32, "nn_conv2d bias")
        if bias.dim() != 1 or bias.shape[0] != O:
            raise ValueError("nn_conv2d bias must be rank-1 of length O")
        flags |= BIAS
        ptrs.append(bias.data_ptr())
        keep.append(bias)
    if residual is not None:
        residual = _req(residual, torch.float32, "nn_conv2d residual")
        if tuple(residual.shape) != (N, O, OH, OW):
            raise ValueError("nn_conv2d residual must have the output shape")
        flags |= RESIDUAL
        ptrs.append(residual.data_ptr())
        keep.append(residual)
    if relu:
        flags |= RELU
    if out is None:
        out = torch.empty((N, O, max(OH, 0), max(OW, 0)), dtype=torch.float32, device=data.device)
    ptrs.append(out.data_ptr())
    desc = Conv2dDesc(N, C, H, W, O, KH, KW, sh, sw, ph, pw, dh, dw, flags, PRECISIONS[precision])
    check("nn_conv2d", load().kxc_b200_nn_conv2d(packed(*ptrs), desc, _stream(data)))
    return out


def nn_conv2d_s8(data, weight, bias, multiplier, shift, strides=(1, 1), padding=(0, 0), dilation=(1, 1), relu=True,
                 simt=False, nhwc=False):
    """int8 convolution, int32 accumulate + bias, fixed-point requantize to int8 (optionally fused relu).

    nhwc=True: data [N,H,W,C], weight [O,KH,KW,C] and the result [N,OH,OW,O] stay in the tensor-core kernel's layout
    (a quantized pipeline's resident activations): no conversion kernels, no workspace. C must be a multiple of the
    kernel's K block (32), except for a stride-2 first layer of <= 8 channels and 64 filters (the image stem), whose
    pixels the library packs to 8 bytes for its direct kernel."""
    data = _req(data, torch.int8, "nn_conv2d_s8 data")
    weight = _req(weight, torch.int8, "nn_conv2d_s8 weight")
    bias = _req(bias, torch.int32, "nn_conv2d_s8 bias")
    multiplier = _req(multiplier, torch.int32, "nn_conv2d_s8 multiplier")
    shift = _req(shift, torch.int32, "nn_conv2d_s8 shift")
    if nhwc:
        N, H, W, C = data.shape
        O, KH, KW, _ = weight.shape
    else:
        N, C, H, W = data.shape
        O, _, KH, KW = weight.shape
    sh, sw = _pair(strides, 1)
    ph, pw = _pair(padding, 0)
    dh, dw = _pair(dilation, 1)
    OH, OW = conv_out_dim(H, KH, sh, ph, dh), conv_out_dim(W, KW, sw, pw, dw)
    out = torch.empty((N, OH, OW, O) if nhwc else (N, O, OH, OW), dtype=torch.int8, device=data.device)
    desc = Conv2dDesc(N, C, H, W, O, KH, KW, sh, sw, ph, pw, dh, dw, BIAS | (RELU if relu else 0) | (NHWC if nhwc else 0),
                      PREC_SIMT if simt else PREC_FP32)
    args = packed(data.data_ptr(), weight.data_ptr(), bias.data_ptr(), multiplier.data_ptr(), shift.data_ptr(),
                  out.data_ptr())
    check("nn_conv2d_s8", load().kxc_b200_nn_conv2d_s8(args, desc, _stream(data)))
    return out


def nn_relu(x):
    x = _req(x, torch.float32, "nn_relu")
    out = torch.empty_like(x)
    check("nn_relu", load().kxc_b200_nn_relu(packed(x.data_ptr(), out.data_ptr()), x.numel(), _stream(x)))
    return out


def add(a, b, relu=False):
    """add(a, b) with right-aligned NumPy broadcasting; relu=True fuses the following nn_relu."""
    a = _req(a, torch.float32, "add lhs")
    b = _req(b, torch.float32, "add rhs")
    if a.dim() > 6 or b.dim() > 6:
        raise ValueError("add: rank must be <= 6")
    desc = AddDesc()
    desc.rank_a, desc.rank_b, desc.relu = a.dim(), b.dim(), int(relu)
    for i, d in enumerate(a.shape):
        desc.shape_a[i] = d
    for i, d in enumerate(b.shape):
        desc.shape_b[i] = d
    out_shape = torch.broadcast_shapes(a.shape, b.shape)
    out = torch.empty(out_shape, dtype=torch.float32, device=a.device)
    check("add", load().kxc_b200_add(packed(a.data_ptr(), b.data_ptr(), out.data_ptr()), desc, _stream(a)))
    return out


def _pool_desc(x, pool_size, strides, padding, ceil_mode, name):
    if x.dim() != 4:
        raise ValueError(f"{name} expects NCHW rank-4 input")
    kh, kw = _pair(pool_size, 1)
    sh, sw = _pair(strides, 1)
    padding = list(padding) if padding is not None else []
    if len(padding) >= 4:
        pt, pl, pb, pr = (int(v) for v in padding[:4])
    elif len(padding) >= 2:
        pt, pl, pb, pr = int(padding[0]), int(padding[1]), int(padding[0]), int(padding[1])
    else:
        pt = pl = pb = pr = 0
    N, C, H, W = x.shape
    OH, OW = pool_out_dim(H, kh, sh, pt, pb, ceil_mode), pool_out_dim(W, kw, sw, pl, pr, ceil_mode)
    return Pool2dDesc(N, C, H, W, kh, kw, sh, sw, pt, pl, pb, pr, int(bool(ceil_mode))), (N, C, max(OH, 0), max(OW, 0))


def nn_max_pool2d(x, pool_size, strides, padding=(0, 0, 0, 0), ceil_mode=False):
    x = _req(x, torch.float32, "nn_max_pool2d")
    desc, oshape = _pool_desc(x, pool_size, strides, padding, ceil_mode, "nn_max_pool2d")
    out = torch.empty(oshape, dtype=torch.float32, device=x.device)
    check("nn_max_pool2d", load().kxc_b200_nn_max_pool2d(packed(x.data_ptr(), out.data_ptr()), desc, _stream(x)))
    return out


def nn_avg_pool2d(x, pool_size, strides, padding=(0, 0, 0, 0), ceil_mode=False):
    x = _req(x, torch.float32, "nn_avg_pool2d")
    desc, oshape = _pool_desc(x, pool_size, strides, padding, ceil_mode, "nn_avg_pool2d")
    out = torch.empty(oshape, dtype=torch.float32, device=x.device)
    check("nn_avg_pool2d", load().kxc_b200_nn_avg_pool2d(packed(x.data_ptr(), out.data_ptr()), desc, _stream(x)))
    return out


def max_pool2d_add_relu(x, residual, pool_size, strides, padding=(0, 0, 0, 0), ceil_mode=False, out=None):
    """nn_max_pool2d -> add(residual) -> nn_relu in one pass."""
    x = _req(x, torch.float32, "max_pool2d_add_relu")
    residual = _req(residual, torch.float32, "max_pool2d_add_relu residual")
    desc, oshape = _pool_desc(x, pool_size, strides, padding, ceil_mode, "max_pool2d_add_relu")
    if tuple(residual.shape) != tuple(oshape):
        raise ValueError("max_pool2d_add_relu: residual must have the pooled shape")
    if out is None:
        out = torch.empty(oshape, dtype=torch.float32, device=x.device)
    check("max_pool2d_add_relu",
          load().kxc_b200_max_pool2d_add_relu(packed(x.data_ptr(), residual.data_ptr(), out.data_ptr()), desc, _stream(x)))
    return out


def nn_global_avg_pool2d(x):
    x = _req(x, torch.float32, "nn_global_avg_pool2d")
    if x.dim() != 4:
        raise ValueError("nn_global_avg_pool2d expects NCHW rank-4 input")
    N, C, H, W = x.shape
    out = torch.empty((N, C, 1, 1), dtype=torch.float32, device=x.device)
    check("nn_global_avg_pool2d",
          load().kxc_b200_nn_global_avg_pool2d(packed(x.data_ptr(), out.data_ptr()), N, C, H, W, _stream(x)))
    return out


def softmax(x, axis=-1):
    """softmax along `axis` (only the last axis: see include/kxc_b200.h)."""
    x = _req(x, torch.float32, "softmax")
    if not 1 <= x.dim() <= 6:
        raise ValueError("softmax expects rank 1..6")
    desc = _lib.SoftmaxDesc(x.dim(), (_lib.i64 * 6)(*x.shape), int(axis))
    out = torch.empty_like(x)
    check("softmax", load().kxc_b200_softmax(packed(x.data_ptr(), out.data_ptr()), desc, _stream(x)))
    return out


def reduce_mean(x, axes, keepdims=True):
    """Mean over `axes`, summed sequentially in the reference's order (bit-exact)."""
    x = _req(x, torch.float32, "reduce_mean")
    if not 1 <= x.dim() <= 6:
        raise ValueError("reduce_mean expects rank 1..6")
    axes = [int(a) for a in axes]
    norm = sorted(a % x.dim() for a in axes)
    oshape = [1 if d in norm else n for d, n in enumerate(x.shape) if keepdims or d not in norm]
    desc = _lib.ReduceDesc(x.dim(), (_lib.i64 * 6)(*x.shape), len(axes), (_lib.i32 * 6)(*axes), 1 if keepdims else 0)
    out = torch.empty(oshape, dtype=torch.float32, device=x.device)
    check("reduce_mean", load().kxc_b200_reduce_mean(packed(x.data_ptr(), out.data_ptr()), desc, _stream(x)))
    return out


_CAST_CODES = {torch.float32: _lib.DT_F32, torch.int32: _lib.DT_I32, torch.int64: _lib.DT_I64, torch.float64: _lib.DT_F64,
               torch.int8: _lib.DT_I8, torch.uint8: _lib.DT_U8}
_CAST_NAMES = {"float32": torch.float32, "int32": torch.int32, "int64": torch.int64, "float64": torch.float64,
               "int8": torch.int8, "uint8": torch.uint8}


def _dev(t, name):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ValueError(f"{name}: expected a CUDA tensor (libkxc_b200 has no CPU path)")
    return t.contiguous()


def matmul(a, b, precision="tf32"):
    """matmul(a[M,K], b[K,N]); rank-2 operands only, like the reference's type inference."""
    a = _req(a, torch.float32, "matmul a")
    b = _req(b, torch.float32, "matmul b")
    if a.dim() != 2 or b.dim() != 2:
        raise ValueError("matmul currently expects rank-2 inputs")
    if a.shape[1] != b.shape[0]:
        raise ValueError("matmul reduction dimension mismatch")
    out = torch.empty((a.shape[0], b.shape[1]), dtype=torch.float32, device=a.device)
    check("matmul", load().kxc_b200_matmul(packed(a.data_ptr(), b.data_ptr(), out.data_ptr()), a.shape[0], b.shape[1],
                                           a.shape[1], PRECISIONS[precision], _stream(a)))
    return out


def transpose(x, axes=None):
    """transpose(x, axes): output dimension i is input dimension axes[i]; no axes reverses the dimensions."""
    x = _dev(x, "transpose")
    if not 1 <= x.dim() <= 6:
        raise ValueError("transpose expects rank 1..6")
    axes = [int(a) for a in axes] if axes else []
    if axes and len(axes) != x.dim():
        raise ValueError("transpose perm rank mismatch")
    norm = [a % x.dim() for a in axes] if axes else list(range(x.dim() - 1, -1, -1))
    if len(set(norm)) != len(norm):
        raise ValueError("transpose duplicate axis")
    out = torch.empty([x.shape[a] for a in norm], dtype=x.dtype, device=x.device)
    desc = _lib.TransposeDesc(x.dim(), (_lib.i64 * 6)(*x.shape), len(axes), (_lib.i32 * 6)(*axes), x.element_size())
    check("transpose", load().kxc_b200_transpose(packed(x.data_ptr(), out.data_ptr()), desc, _stream(x)))
    return out


def reshape_out_shape(in_shape, newshape, allowzero=False):
    """The output shape ReshapeInferType derives (src/relay/type_infer.cc:454-512): positive entries as given, 0 copies
    the input's extent at that position unless allowzero, one -1 is inferred from the element count."""
    in_shape = [int(d) for d in in_shape]
    total = 1
    for d in in_shape:
        total *= d
    out, infer, known = [], -1, 1
    for i, dim in enumerate(int(d) for d in newshape):
        if dim > 0:
            out.append(dim)
            known *= dim
        elif dim == 0:
            if allowzero:
                out.append(0)
                known = 0
            else:
                if i >= len(in_shape):
                    raise ValueError("reshape 0-dim copy index exceeds input rank")
                out.append(in_shape[i])
                known *= in_shape[i]
        elif dim == -1:
            if infer >= 0:
                raise ValueError("reshape allows at most one inferred -1 dimension")
            infer = len(out)
            out.append(-1)
        else:
            raise ValueError("reshape only supports positive, 0, and -1 dimensions")
    if infer >= 0 and known > 0:
        if total % known != 0:
            raise ValueError("reshape cannot infer -1 dimension from element count")
        out[infer] = total // known
    elif infer < 0 and total != known:
        raise ValueError("reshape element count mismatch")
    return out


def reshape(x, newshape, allowzero=False):
    x = _dev(x, "reshape")
    out = torch.empty(reshape_out_shape(x.shape, newshape, allowzero), dtype=x.dtype, device=x.device)
    check("reshape", load().kxc_b200_reshape(packed(x.data_ptr(), out.data_ptr()), x.numel(), x.element_size(), _stream(x)))
    return out


def cast(x, dtype):
    """cast(x, dtype): dtype is a torch dtype or the reference's dtype name ("float32", "int32", "int64", "float64",
    "int8", "uint8"); bool is refused by the library."""
    x = _dev(x, "cast")
    if isinstance(dtype, str):
        if dtype == "bool":
            to, tdt = _lib.DT_BOOL, torch.bool
        elif dtype not in _CAST_NAMES:
            raise ValueError(f"cast has unsupported dtype: {dtype}")
        else:
            tdt = _CAST_NAMES[dtype]
            to = _CAST_CODES[tdt]
    else:
        tdt = dtype
        to = _lib.DT_BOOL if dtype == torch.bool else _CAST_CODES.get(dtype, -1)
    frm = _lib.DT_BOOL if x.dtype == torch.bool else _CAST_CODES.get(x.dtype, -1)
    out = torch.empty(x.shape, dtype=tdt, device=x.device)
    check("cast", load().kxc_b200_cast(packed(x.data_ptr(), out.data_ptr()), x.numel(), frm, to, _stream(x)))
    return out


def nn_flatten(x):
    x = _req(x, torch.float32, "nn_flatten")
    out = torch.empty((x.shape[0], x.numel() // max(x.shape[0], 1)), dtype=torch.float32, device=x.device)
    check("nn_flatten", load().kxc_b200_nn_flatten(packed(x.data_ptr(), out.data_ptr()), x.numel(), _stream(x)))
    return out


def nn_dense(data, weight, precision="tf32"):
    data = _req(data, torch.float32, "nn_dense data")
    weight = _req(weight, torch.float32, "nn_dense weight")
    M, K = data.shape
    Nn, K2 = weight.shape
    if K != K2:
        raise ValueError("nn_dense: inner dimensions differ")
    out = torch.empty((M, Nn), dtype=torch.float32, device=data.device)
    desc = GemmDesc(M, Nn, K, 1.0, 1.0, 0, 1, 0, PRECISIONS[precision])
    check("nn_dense", load().kxc_b200_nn_gemm(packed(data.data_ptr(), weight.data_ptr(), out.data_ptr()), desc, _stream(data)))
    return out


def nn_gemm(a, b, c, alpha=1.0, beta=1.0, transA=0, transB=0, precision="tf32"):
    a = _req(a, torch.float32, "nn_gemm A")
    b = _req(b, torch.float32, "nn_gemm B")
    c = _req(c, torch.float32, "nn_gemm C")
    M, K = a.shape
    Nn = b.shape[0] if transB else b.shape[1]
    out = torch.empty((M, Nn), dtype=torch.float32, device=a.device)
    desc = GemmDesc(M, Nn, K, float(alpha), float(beta), int(transA), int(transB), 1, PRECISIONS[precision])
    check("nn_gemm", load().kxc_b200_nn_gemm(packed(a.data_ptr(), b.data_ptr(), c.data_ptr(), out.data_ptr()), desc, _stream(a)))
    return out


def device_status(device=None):
    """Synchronise the current stream and raise if a tensor-core kernel gave up a bounded wait."""
    import ctypes
    st = ctypes.c_int32(0)
    stream = torch.cuda.current_stream(device).cuda_stream
    check("device_status", load().kxc_b200_device_status(stream, ctypes.byref(st)))
    return st.value

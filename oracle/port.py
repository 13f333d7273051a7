"""numpy-facing binding of the plain-C oracle port (kxc_oracle.c). TEST INFRASTRUCTURE ONLY."""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libkxc_oracle.so")
_lib = None

i64 = ctypes.c_int64
i32 = ctypes.c_int32
vp = ctypes.c_void_p


def build(force=False):
    src = os.path.join(_HERE, "kxc_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "port"])
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.kxc_oracle_conv_out_dim.restype = i64
        _lib.kxc_oracle_conv_out_dim.argtypes = [i64] * 5
        _lib.kxc_oracle_pool_out_dim.restype = i64
        _lib.kxc_oracle_pool_out_dim.argtypes = [i64] * 5 + [i32]
        _lib.kxc_oracle_requant_one.restype = ctypes.c_int8
        _lib.kxc_oracle_requant_one.argtypes = [i32] * 4
        _lib.kxc_oracle_conv2d_f32.argtypes = [vp] * 4 + [i64] * 13
        _lib.kxc_oracle_conv2d_i32.argtypes = [vp] * 4 + [i64] * 13
        _lib.kxc_oracle_conv2d_s8_requant.argtypes = [vp] * 5 + [i32] + [vp] * 2 + [i64] * 13
        _lib.kxc_oracle_relu_f32.argtypes = [vp, vp, i64]
        _lib.kxc_oracle_add_f32.argtypes = [vp, vp, vp, vp, vp, vp, i32]
        _lib.kxc_oracle_max_pool2d_f32.argtypes = [vp, vp] + [i64] * 12 + [i32]
        _lib.kxc_oracle_avg_pool2d_f32.argtypes = [vp, vp] + [i64] * 12 + [i32]
        _lib.kxc_oracle_global_avg_pool2d_f32.argtypes = [vp, vp] + [i64] * 4
        _lib.kxc_oracle_dense_f32.argtypes = [vp, vp, vp] + [i64] * 3
        _lib.kxc_oracle_softmax_f32.argtypes = [vp, vp] + [i64] * 3
        _lib.kxc_oracle_reduce_mean_f32.argtypes = [vp, vp, i32, vp, vp]
        _lib.kxc_oracle_matmul_f32.argtypes = [vp, vp, vp] + [i64] * 3
        _lib.kxc_oracle_transpose.argtypes = [vp, vp, i32, vp, vp, i32]
        _lib.kxc_oracle_cast.argtypes = [vp, vp, i64, i32, i32]
        _lib.kxc_oracle_gemm_f32.argtypes = [vp] * 4 + [i64] * 3 + [ctypes.c_float] * 2 + [i32] * 2
        _lib.kxc_oracle_round_bf16.argtypes = [vp, vp, i64]
        _lib.kxc_oracle_round_tf32.argtypes = [vp, vp, i64]
        for name in ("round_bf16", "round_tf32"):
            getattr(_lib, "kxc_oracle_" + name).restype = None
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(vp)


def _c(a, dt):
    return None if a is None else np.ascontiguousarray(a, dtype=dt)


def _check(rc, what):
    if rc != 0:
        raise RuntimeError(f"oracle {what} returned error code {rc}")


def conv_out_dim(n, k, s, p, d=1):
    return int(lib().kxc_oracle_conv_out_dim(n, k, s, p, d))


def pool_out_dim(n, k, s, p0, p1, ceil_mode=False):
    return int(lib().kxc_oracle_pool_out_dim(n, k, s, p0, p1, int(ceil_mode)))


def _conv_generic(fn, dt, data, weight, bias, stride, pad, dilation):
    data, weight, bias = _c(data, dt), _c(weight, dt), _c(bias, dt)
    N, C, H, W = data.shape
    O, C2, KH, KW = weight.shape
    assert C == C2
    OH = conv_out_dim(H, KH, stride[0], pad[0], dilation[0])
    OW = conv_out_dim(W, KW, stride[1], pad[1], dilation[1])
    out = np.empty((N, O, OH, OW), dtype=dt)
    _check(fn(_p(data), _p(weight), _p(bias), _p(out), N, C, H, W, O, KH, KW, stride[0], stride[1], pad[0], pad[1],
              dilation[0], dilation[1]), "conv2d")
    return out


def conv2d(data, weight, bias=None, stride=(1, 1), pad=(0, 0), dilation=(1, 1)):
    return _conv_generic(lib().kxc_oracle_conv2d_f32, np.float32, data, weight, bias, stride, pad, dilation)


def conv2d_i32(data, weight, bias=None, stride=(1, 1), pad=(0, 0), dilation=(1, 1)):
    return _conv_generic(lib().kxc_oracle_conv2d_i32, np.int32, data, weight, bias, stride, pad, dilation)


def conv2d_s8_requant(data, weight, bias, multiplier, shift, relu=True, stride=(1, 1), pad=(0, 0), dilation=(1, 1),
                      return_acc=False):
    data, weight = _c(data, np.int8), _c(weight, np.int8)
    bias, multiplier, shift = _c(bias, np.int32), _c(multiplier, np.int32), _c(shift, np.int32)
    N, C, H, W = data.shape
    O, _, KH, KW = weight.shape
    OH = conv_out_dim(H, KH, stride[0], pad[0], dilation[0])
    OW = conv_out_dim(W, KW, stride[1], pad[1], dilation[1])
    out = np.empty((N, O, OH, OW), dtype=np.int8)
    acc = np.empty((N, O, OH, OW), dtype=np.int32) if return_acc else None
    _check(lib().kxc_oracle_conv2d_s8_requant(_p(data), _p(weight), _p(bias), _p(multiplier), _p(shift), int(relu),
                                              _p(out), _p(acc), N, C, H, W, O, KH, KW, stride[0], stride[1], pad[0],
                                              pad[1], dilation[0], dilation[1]), "conv2d_s8_requant")
    return (out, acc) if return_acc else out


def requant_one(acc, multiplier, shift, relu=True):
    return int(lib().kxc_oracle_requant_one(int(acc), int(multiplier), int(shift), int(relu)))


def relu(x):
    x = _c(x, np.float32)
    out = np.empty_like(x)
    _check(lib().kxc_oracle_relu_f32(_p(x), _p(out), x.size), "relu")
    return out


def add(a, b):
    a, b = _c(a, np.float32), _c(b, np.float32)
    rank = max(a.ndim, b.ndim, 1)
    ash = (1,) * (rank - a.ndim) + a.shape
    bsh = (1,) * (rank - b.ndim) + b.shape
    osh = tuple(y if x == 1 else x for x, y in zip(ash, bsh))
    out = np.empty(osh, dtype=np.float32)
    A = np.array(ash, dtype=np.int64)
    B = np.array(bsh, dtype=np.int64)
    Osh = np.array(osh, dtype=np.int64)
    _check(lib().kxc_oracle_add_f32(_p(a), _p(A), _p(b), _p(B), _p(out), _p(Osh), rank), "add")
    return out


def _pool(fn, x, ksize, stride, pad, ceil_mode):
    x = _c(x, np.float32)
    N, C, H, W = x.shape
    if len(pad) == 2:
        pad = (pad[0], pad[1], pad[0], pad[1])
    OH = pool_out_dim(H, ksize[0], stride[0], pad[0], pad[2], ceil_mode)
    OW = pool_out_dim(W, ksize[1], stride[1], pad[1], pad[3], ceil_mode)
    out = np.empty((N, C, OH, OW), dtype=np.float32)
    _check(fn(_p(x), _p(out), N, C, H, W, ksize[0], ksize[1], stride[0], stride[1], pad[0], pad[1], pad[2], pad[3],
              int(ceil_mode)), "pool2d")
    return out


def max_pool2d(x, ksize, stride, pad=(0, 0, 0, 0), ceil_mode=False):
    return _pool(lib().kxc_oracle_max_pool2d_f32, x, ksize, stride, pad, ceil_mode)


def avg_pool2d(x, ksize, stride, pad=(0, 0, 0, 0), ceil_mode=False):
    return _pool(lib().kxc_oracle_avg_pool2d_f32, x, ksize, stride, pad, ceil_mode)


def global_avg_pool2d(x):
    x = _c(x, np.float32)
    N, C, H, W = x.shape
    out = np.empty((N, C, 1, 1), dtype=np.float32)
    _check(lib().kxc_oracle_global_avg_pool2d_f32(_p(x), _p(out), N, C, H, W), "global_avg_pool2d")
    return out


def softmax(x, axis=-1):
    """src/relay/op/nn/softmax.cc:44-70. Last axis only: for an inner axis the reference's keepdims reduction
    (include/te/topi/reduction.h:47-58) indexes elements of other rows, which nothing should reproduce."""
    x = _c(x, np.float32)
    axis = axis % x.ndim
    if axis != x.ndim - 1:
        raise ValueError("softmax: only the last axis (see the docstring)")
    outer = int(np.prod(x.shape[:axis], dtype=np.int64))
    inner = int(np.prod(x.shape[axis + 1:], dtype=np.int64))
    out = np.empty_like(x)
    _check(lib().kxc_oracle_softmax_f32(_p(x), _p(out), outer, x.shape[axis], inner), "softmax")
    return out


def reduce_mean(x, axes, keepdims=True):
    """src/relay/op/tensor/reduce.cc:81-99. keepdims only for trailing reduced axes (same reference defect as softmax)."""
    x = _c(x, np.float32)
    axes = sorted(a % x.ndim for a in axes)
    if keepdims and axes != list(range(x.ndim - len(axes), x.ndim)):
        raise ValueError("reduce_mean: keepdims needs the reduced axes to be the trailing ones (see the docstring)")
    shape = np.asarray(x.shape, dtype=np.int64)
    flags = np.asarray([1 if d in axes else 0 for d in range(x.ndim)], dtype=np.int32)
    out_shape = [1 if d in axes else n for d, n in enumerate(x.shape) if keepdims or d not in axes]
    out = np.empty(out_shape, dtype=np.float32)
    _check(lib().kxc_oracle_reduce_mean_f32(_p(x), _p(out), x.ndim, _p(shape), _p(flags)), "reduce_mean")
    return out


CAST_CODES = {np.dtype(np.float32): 0, np.dtype(np.int32): 1, np.dtype(np.int64): 2, np.dtype(np.float64): 3,
              np.dtype(np.int8): 5, np.dtype(np.uint8): 6}


def matmul(a, b):
    """include/te/topi/nn.h:82-101: a[M,K] x b[K,N], k ascending."""
    a, b = _c(a, np.float32), _c(b, np.float32)
    M, K = a.shape
    Nn = b.shape[1]
    out = np.empty((M, Nn), dtype=np.float32)
    _check(lib().kxc_oracle_matmul_f32(_p(a), _p(b), _p(out), M, Nn, K), "matmul")
    return out


def transpose(x, axes=None):
    """include/te/topi/transform.h:20-52; no axes reverses the dimensions."""
    x = np.ascontiguousarray(x)
    perm = [a % x.ndim for a in axes] if axes else list(range(x.ndim - 1, -1, -1))
    out = np.empty([x.shape[a] for a in perm], dtype=x.dtype)
    if x.size:
        shape = np.asarray(x.shape, dtype=np.int64)
        permv = np.asarray(perm, dtype=np.int32)
        _check(lib().kxc_oracle_transpose(_p(x), _p(out), x.ndim, _p(shape), _p(permv), x.dtype.itemsize), "transpose")
    return out


def reshape(x, out_shape):
    """src/relay/op/tensor/transform.cc:185-204: the flat order is kept."""
    return np.ascontiguousarray(x).reshape(out_shape).copy()


def cast(x, dtype):
    """include/te/topi/elemwise.h:113-122 with CodeGenLLVM::CastValue's scalar rule (src/codegen/codegen_llvm.cc:219-248)."""
    x = np.ascontiguousarray(x)
    out = np.empty(x.shape, dtype=dtype)
    _check(lib().kxc_oracle_cast(_p(x), _p(out), x.size, CAST_CODES[x.dtype], CAST_CODES[out.dtype]), "cast")
    return out


def dense(a, b):
    a, b = _c(a, np.float32), _c(b, np.float32)
    M, K = a.shape
    Nn = b.shape[0]
    out = np.empty((M, Nn), dtype=np.float32)
    _check(lib().kxc_oracle_dense_f32(_p(a), _p(b), _p(out), M, Nn, K), "dense")
    return out


def gemm(a, b, c, alpha=1.0, beta=1.0, transA=0, transB=1):
    a, b, c = _c(a, np.float32), _c(b, np.float32), _c(c, np.float32)
    M, K = a.shape
    Nn = b.shape[0] if transB else b.shape[1]
    out = np.empty((M, Nn), dtype=np.float32)
    _check(lib().kxc_oracle_gemm_f32(_p(a), _p(b), _p(c), _p(out), M, Nn, K, alpha, beta, transA, transB), "gemm")
    return out


def round_bf16(x):
    x = _c(x, np.float32)
    out = np.empty_like(x)
    lib().kxc_oracle_round_bf16(_p(x), _p(out), x.size)
    return out


def round_tf32(x):
    x = _c(x, np.float32)
    out = np.empty_like(x)
    lib().kxc_oracle_round_tf32(_p(x), _p(out), x.size)
    return out

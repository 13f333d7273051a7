"""ctypes binding of libkxc_b200.so (C ABI: include/kxc_b200.h)."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_NAME = "libkxc_b200.so"
_lib = None

i32 = ctypes.c_int32
i64 = ctypes.c_int64
vp = ctypes.c_void_p
vpp = ctypes.POINTER(ctypes.c_void_p)

OK = 0
BIAS, RESIDUAL, RELU, NHWC = 1, 2, 4, 8
PREC_FP32, PREC_TF32, PREC_BF16, PREC_SIMT, PREC_TF32X3 = 0, 1, 2, 3, 4
# cast dtype codes: the reference's CastAttrs codes (src/relay/op/tensor/transform.cc:84-103)
DT_F32, DT_I32, DT_I64, DT_F64, DT_BOOL, DT_I8, DT_U8 = 0, 1, 2, 3, 4, 5, 6


class KxcError(RuntimeError):
    """Raised when an entry point returns non-zero (the reference raises
    'Kernel <name> returned error code N', src/codegen/compiled_kernel.cc:50-54)."""

    def __init__(self, name, code, message):
        super().__init__(f"Kernel {name} returned error code {code}: {message}")
        self.code = code


class Conv2dDesc(ctypes.Structure):
    _fields_ = [(n, i32) for n in ("n", "c", "h", "w", "o", "kh", "kw", "stride_h", "stride_w", "pad_h", "pad_w",
                                   "dilation_h", "dilation_w", "flags", "precision")]


class AddDesc(ctypes.Structure):
    _fields_ = [("rank_a", i32), ("rank_b", i32), ("shape_a", i64 * 6), ("shape_b", i64 * 6), ("relu", i32)]


class SoftmaxDesc(ctypes.Structure):
    _fields_ = [("rank", i32), ("shape", i64 * 6), ("axis", i32)]


class ReduceDesc(ctypes.Structure):
    _fields_ = [("rank", i32), ("shape", i64 * 6), ("num_axes", i32), ("axes", i32 * 6), ("keepdims", i32)]


class TransposeDesc(ctypes.Structure):
    _fields_ = [("rank", i32), ("shape", i64 * 6), ("num_axes", i32), ("perm", i32 * 6), ("elem_bytes", i32)]


class Pool2dDesc(ctypes.Structure):
    _fields_ = [(n, i32) for n in ("n", "c", "h", "w", "kh", "kw", "stride_h", "stride_w", "pad_top", "pad_left",
                                   "pad_bottom", "pad_right", "ceil_mode")]


class GemmDesc(ctypes.Structure):
    _fields_ = [("m", i32), ("n", i32), ("k", i32), ("alpha", ctypes.c_float), ("beta", ctypes.c_float),
                ("transA", i32), ("transB", i32), ("has_c", i32), ("precision", i32)]


# every symbol include/kxc_b200.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "kxc_b200_last_error": (ctypes.c_char_p, []),
    "kxc_b200_abi_version": (i32, []),
    "kxc_b200_device_check": (i32, []),
    "kxc_b200_device_status": (i32, [vp, ctypes.POINTER(i32)]),
    "kxc_b200_selftest_bounded_wait": (i32, [i64, vp, ctypes.POINTER(i32)]),
    "kxc_b200_selftest_per_device_once": (i32, []),
    "kxc_b200_nn_conv2d": (i32, [vpp, ctypes.POINTER(Conv2dDesc), vp]),
    "kxc_b200_nn_conv2d_s8": (i32, [vpp, ctypes.POINTER(Conv2dDesc), vp]),
    "kxc_b200_nn_conv2d_static_scratch": (i32, [vpp, ctypes.POINTER(Conv2dDesc), vp]),
    "kxc_b200_static_scratch_bytes": (i64, []),
    "kxc_b200_nn_relu": (i32, [vpp, i64, vp]),
    "kxc_b200_add": (i32, [vpp, ctypes.POINTER(AddDesc), vp]),
    "kxc_b200_nn_max_pool2d": (i32, [vpp, ctypes.POINTER(Pool2dDesc), vp]),
    "kxc_b200_nn_avg_pool2d": (i32, [vpp, ctypes.POINTER(Pool2dDesc), vp]),
    "kxc_b200_max_pool2d_add_relu": (i32, [vpp, ctypes.POINTER(Pool2dDesc), vp]),
    "kxc_b200_nn_global_avg_pool2d": (i32, [vpp, i32, i32, i32, i32, vp]),
    "kxc_b200_softmax": (i32, [vpp, ctypes.POINTER(SoftmaxDesc), vp]),
    "kxc_b200_reduce_mean": (i32, [vpp, ctypes.POINTER(ReduceDesc), vp]),
    "kxc_b200_matmul": (i32, [vpp, i32, i32, i32, i32, vp]),
    "kxc_b200_transpose": (i32, [vpp, ctypes.POINTER(TransposeDesc), vp]),
    "kxc_b200_reshape": (i32, [vpp, i64, i32, vp]),
    "kxc_b200_cast": (i32, [vpp, i64, i32, i32, vp]),
    "kxc_b200_nn_flatten": (i32, [vpp, i64, vp]),
    "kxc_b200_nn_gemm": (i32, [vpp, ctypes.POINTER(GemmDesc), vp]),
}


def library_path():
    return os.path.join(_HERE, _LIB_NAME)


def load():
    """Load the CUDA library; there is no fallback when it is missing."""
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise ImportError(f"{path} is not built: run `python -c 'import __graft_entry__ as g; g.build()'` "
                              f"or `make -C hdkx_aicompiler_b200/csrc` (needs nvcc with sm_100a)")
        lib = ctypes.CDLL(path)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def last_error():
    msg = load().kxc_b200_last_error()
    return msg.decode(errors="replace") if msg else ""


def check(name, rc):
    if rc != OK:
        raise KxcError(name, rc, last_error())


def packed(*ptrs):
    """void** packed_args from raw addresses."""
    return (ctypes.c_void_p * len(ptrs))(*ptrs)

"""The reference compiler's own CPU lowering as a checker. TEST INFRASTRUCTURE ONLY.

oracle/_ref/ref_emit (built by `make -C oracle ref` from the reference's unmodified sources) lowers a
small Relay graph to C text through the reference's Relay -> TE -> TIR -> CodeGenC pipeline. This
module compiles that text with `gcc -O3 -march=native -ffp-contract=off` (FMA contraction off: the
reference's LLVM backend emits separate fmul/fadd) and calls the resulting
`int32_t f(void** packed_args)` with numpy buffers, inputs first and the output last, the ABI of
src/codegen/compiled_kernel.cc:41-55.

Intermediate tensors are stack arrays in the emitted C (src/codegen/codegen_c.cc:220-232); they are
rewritten to malloc/free, which is what the LLVM backend does (src/codegen/codegen_llvm.cc:591-616).

Nothing here reads the reference checkout at run time: ref_emit is a self-contained binary and gcc is
part of the image, so kernels for new shapes can be generated on any box that has oracle/_ref/.
"""
import ctypes
import hashlib
import os
import re
import subprocess
import threading

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_EMIT = os.path.join(_HERE, "_ref", "ref_emit")
_lock = threading.Lock()
_cache = {}

_DT = {"float32": np.float32, "int32": np.int32}


def available():
    return os.path.exists(_EMIT) and os.access(_EMIT, os.X_OK)


def _cpu_tag():
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return hashlib.sha1(line.encode()).hexdigest()[:10]
    except OSError:
        pass
    return "generic"


_VLA = re.compile(r"^  (float|int32_t|double|int64_t|int8_t|uint8_t) ([A-Za-z_0-9]+)\[(.*)\];$", re.M)


def _heapify(src):
    names = []

    def sub(m):
        names.append(m.group(2))
        return f"  {m.group(1)}* {m.group(2)} = ({m.group(1)}*)malloc(sizeof({m.group(1)}) * (size_t)({m.group(3)}));"

    src = _VLA.sub(sub, src)
    if names:
        frees = "".join(f"  free({n});\n" for n in names)
        idx = src.rfind("  return 0;")
        src = src[:idx] + frees + src[idx:]
    return src


def kernel(program):
    """Compile (once) and return the C entry point for a ref_emit program string."""
    with _lock:
        fn = _cache.get(program)
        if fn is not None:
            return fn
        if not available():
            raise RuntimeError("oracle/_ref/ref_emit is not built (make -C oracle ref)")
        tag = _cpu_tag()
        key = hashlib.sha1(program.encode()).hexdigest()[:20]
        kdir = os.path.join(_HERE, "_ref", "kernels", tag)
        os.makedirs(kdir, exist_ok=True)
        so = os.path.join(kdir, f"k_{key}.so")
        if not os.path.exists(so):
            sym = "kxc_ref_kernel"
            res = subprocess.run([_EMIT, sym, program], capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"ref_emit failed for {program!r}: {res.stderr.strip()}")
            csrc = os.path.join(kdir, f"k_{key}.c")
            with open(csrc, "w") as f:
                f.write(_heapify(res.stdout))
            tmp = so + f".tmp{os.getpid()}"
            subprocess.check_call(["gcc", "-O3", "-march=native", "-ffp-contract=off", "-fno-fast-math", "-w", "-Dcast(x)=(x)",
                                   "-shared", "-fPIC", csrc, "-o", tmp, "-lm"])
            os.replace(tmp, so)
        lib = ctypes.CDLL(so)
        fn = lib.kxc_ref_kernel
        fn.restype = ctypes.c_int32
        fn.argtypes = [ctypes.POINTER(ctypes.c_void_p)]
        _cache[program] = fn
        return fn


def run(program, inputs, out_shape, out_dtype=np.float32):
    fn = kernel(program)
    bufs = [np.ascontiguousarray(a) for a in inputs]
    out = np.empty(out_shape, dtype=out_dtype)
    args = (ctypes.c_void_p * (len(bufs) + 1))(*[b.ctypes.data for b in bufs], out.ctypes.data)
    rc = fn(args)
    if rc != 0:
        raise RuntimeError(f"Kernel returned error code {rc}")
    return out


def _shape(a):
    return ",".join(str(int(d)) for d in a.shape)


def _dtn(a):
    return {np.dtype(np.float32): "float32", np.dtype(np.int32): "int32"}[a.dtype]


def _out_dim(n, k, s, p, d):
    return (n + 2 * p - ((k - 1) * d + 1)) // s + 1


def conv2d(data, weight, bias=None, stride=(1, 1), pad=(0, 0), dilation=(1, 1), relu=False):
    """nn_conv2d (+bias) (+nn_relu) in one lowered function, like the reference's unfused PrimFunc."""
    dt = _dtn(data)
    prog = f"in data {dt} {_shape(data)};in w {dt} {_shape(weight)};"
    ins = [data, weight]
    if bias is not None:
        prog += f"in b {dt} {_shape(bias)};"
        ins.append(bias)
    prog += (f"conv2d c data w {'b' if bias is not None else '-'} {stride[0]},{stride[1]} {pad[0]},{pad[1]} "
             f"{dilation[0]},{dilation[1]}")
    if relu:
        prog += ";relu r c"
    N, C, H, W = data.shape
    O, _, KH, KW = weight.shape
    OH = _out_dim(H, KH, stride[0], pad[0], dilation[0])
    OW = _out_dim(W, KW, stride[1], pad[1], dilation[1])
    return run(prog, ins, (N, O, OH, OW), data.dtype)


def relu(x):
    return run(f"in x {_dtn(x)} {_shape(x)};relu r x", [x], x.shape, x.dtype)


def add(a, b):
    out_shape = np.broadcast_shapes(a.shape, b.shape)
    return run(f"in a {_dtn(a)} {_shape(a)};in b {_dtn(b)} {_shape(b)};add s a b", [a, b], out_shape, a.dtype)


def _pool(kind, x, ksize, stride, pad, ceil_mode):
    if len(pad) == 2:
        pad = (pad[0], pad[1], pad[0], pad[1])
    N, C, H, W = x.shape

    def od(n, k, s, p0, p1):
        num = n + p0 + p1 - k
        return (num + s - 1) // s + 1 if ceil_mode else num // s + 1

    OH, OW = od(H, ksize[0], stride[0], pad[0], pad[2]), od(W, ksize[1], stride[1], pad[1], pad[3])
    prog = (f"in x float32 {_shape(x)};{kind} p x {ksize[0]},{ksize[1]} {stride[0]},{stride[1]} "
            f"{pad[0]},{pad[1]},{pad[2]},{pad[3]} {int(ceil_mode)}")
    return run(prog, [x], (N, C, OH, OW))


def max_pool2d(x, ksize, stride, pad=(0, 0, 0, 0), ceil_mode=False):
    return _pool("max_pool2d", x, ksize, stride, pad, ceil_mode)


def avg_pool2d(x, ksize, stride, pad=(0, 0, 0, 0), ceil_mode=False):
    return _pool("avg_pool2d", x, ksize, stride, pad, ceil_mode)


def global_avg_pool2d(x):
    N, C, _, _ = x.shape
    return run(f"in x float32 {_shape(x)};global_avg_pool2d p x", [x], (N, C, 1, 1))


def softmax(x, axis=-1):
    return run(f"in x float32 {_shape(x)};softmax p x {axis % x.ndim}", [x], x.shape)


def reduce_mean(x, axes, keepdims=True):
    axes = sorted(a % x.ndim for a in axes)
    out_shape = [1 if d in axes else n for d, n in enumerate(x.shape) if keepdims or d not in axes]
    return run(f"in x float32 {_shape(x)};reduce_mean p x {','.join(map(str, axes))} {1 if keepdims else 0}", [x], out_shape)


_NAMES = {np.dtype(np.float32): "float32", np.dtype(np.int32): "int32", np.dtype(np.int64): "int64",
          np.dtype(np.float64): "float64", np.dtype(np.int8): "int8", np.dtype(np.uint8): "uint8"}
_CAST_CODES = {"float32": 0, "int32": 1, "int64": 2, "float64": 3, "int8": 5, "uint8": 6}


def matmul(a, b):
    return run(f"in a float32 {_shape(a)};in b float32 {_shape(b)};matmul m a b", [a, b], (a.shape[0], b.shape[1]))


def transpose(x, axes=None):
    perm = [a % x.ndim for a in axes] if axes else list(range(x.ndim - 1, -1, -1))
    spec = ",".join(str(int(a)) for a in axes) if axes else "-"
    return run(f"in x {_NAMES[x.dtype]} {_shape(x)};transpose t x {spec}", [x], [x.shape[a] for a in perm], x.dtype)


def reshape(x, newshape, out_shape):
    """`newshape` as the attribute holds it (0 and -1 allowed); `out_shape` is the resolved shape of the result."""
    spec = ",".join(str(int(d)) for d in newshape)
    return run(f"in x {_NAMES[x.dtype]} {_shape(x)};reshape r x {spec}", [x], out_shape, x.dtype)


def cast(x, dtype):
    """The generated C calls `cast(v)`, which CodeGenC leaves undefined (src/codegen/codegen_c.cc:155-169); kernel()
    compiles with -Dcast(x)=(x), so the conversion is the assignment's, i.e. what CodeGenLLVM::CastValue emits."""
    dtype = np.dtype(dtype)
    return run(f"in x {_NAMES[x.dtype]} {_shape(x)};cast c x {_CAST_CODES[_NAMES[dtype]]}", [x], x.shape, dtype)


def dense(a, b):
    return run(f"in a float32 {_shape(a)};in b float32 {_shape(b)};dense d a b", [a, b], (a.shape[0], b.shape[0]))


def gemm(a, b, c, alpha=1.0, beta=1.0, transA=0, transB=1):
    Nn = b.shape[0] if transB else b.shape[1]
    prog = (f"in a float32 {_shape(a)};in b float32 {_shape(b)};in c float32 {_shape(c)};"
            f"gemm g a b c {alpha!r} {beta!r} {transA} {transB}")
    return run(prog, [a, b, c], (a.shape[0], Nn))


def pool_add_relu(x, res, ksize=(3, 3), stride=(2, 2), pad=(1, 1, 1, 1)):
    """The memory-bound chain max_pool2d -> add(residual) -> relu as ONE lowered reference function."""
    N, C, H, W = x.shape
    OH = (H + pad[0] + pad[2] - ksize[0]) // stride[0] + 1
    OW = (W + pad[1] + pad[3] - ksize[1]) // stride[1] + 1
    prog = (f"in x float32 {_shape(x)};in res float32 {_shape(res)};"
            f"max_pool2d p x {ksize[0]},{ksize[1]} {stride[0]},{stride[1]} {pad[0]},{pad[1]},{pad[2]},{pad[3]} 0;"
            f"add s p res;relu r s")
    return run(prog, [x, res], (N, C, OH, OW))

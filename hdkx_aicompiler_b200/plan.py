"""Whole-graph execution through kxc_b200_plan_* (include/kxc_b200_plan.h).

`CompiledGraph` plays the role of the reference's `CompiledModule` for one Relay function
(src/api/compiler.cc:149-168): `run(input)` launches the graph with the packed argument list
inputs ++ constants (lowering order) ++ output and returns the output tensor.

Precisions and what they cost in accuracy, measured on ResNet-18 with the benchmark's synthetic weights (logits of
magnitude ~300) against the reference's fp32 arithmetic, worst element of the logits:

    "fp32"    CUDA cores in the reference's operation order            bit-identical
    "tf32x3"  three tf32 tensor-core passes per contraction            8e-2 absolute, 2.6e-4 of the logit scale
    "tf32"    one pass, operands rounded to tf32                       1.7e-1 absolute, 5.2e-4 of the logit scale
    "bf16"    bf16 activations and weights, fp32 accumulate            1.4 absolute, 4.2e-3 of the logit scale

"tf32x3" removes the operand rounding (a single layer then agrees to ~2e-5), but not the rounding inside the tensor
core's own fp32 accumulation, which truncates as it aligns the partial products of a long reduction; over twenty
layers that is what remains, so only "fp32" reproduces the reference to the last bits.
"""
import ctypes

import torch

from . import _lib, relay
from ._lib import PREC_BF16, PREC_FP32, PREC_TF32, check, i32, i64, load, packed, vp, vpp

PRECISIONS = {"bf16": PREC_BF16, "tf32": PREC_TF32, "fp32": PREC_FP32, "tf32x3": _lib.PREC_TF32X3}


class Conv2dAttrsC(ctypes.Structure):
    _fields_ = [("strides", i32 * 2), ("padding", i32 * 2), ("dilation", i32 * 2), ("groups", i32)]


class Pool2dAttrsC(ctypes.Structure):
    _fields_ = [("pool_size", i32 * 2), ("strides", i32 * 2), ("padding", i32 * 4), ("ceil_mode", i32)]


class GemmAttrsC(ctypes.Structure):
    _fields_ = [("alpha", ctypes.c_float), ("beta", ctypes.c_float), ("transA", i32), ("transB", i32)]


class SoftmaxAttrsC(ctypes.Structure):
    _fields_ = [("axis", i32)]


class FlattenAttrsC(ctypes.Structure):
    _fields_ = [("axis", i32)]


_PLAN_SYMBOLS = {
    "kxc_b200_plan_create": (i32, [i32, ctypes.POINTER(vp)]),
    "kxc_b200_plan_destroy": (i32, [vp]),
    "kxc_b200_plan_add_input": (i32, [vp, i32, i32, ctypes.POINTER(i64)]),
    "kxc_b200_plan_add_constant": (i32, [vp, i32, i32, ctypes.POINTER(i64)]),
    "kxc_b200_plan_add_kernel": (i32, [vp, ctypes.c_char_p, vp, i32, ctypes.POINTER(i32), i32]),
    "kxc_b200_plan_set_output": (i32, [vp, i32]),
    "kxc_b200_plan_finalize": (i32, [vp]),
    "kxc_b200_plan_value_shape": (i32, [vp, i32, ctypes.POINTER(i64)]),
    "kxc_b200_plan_num_launches": (i32, [vp]),
    "kxc_b200_plan_run": (i32, [vp, vpp, vp]),
    "kxc_b200_plan_set_cuda_graph": (i32, [vp, i32]),
    "kxc_b200_plan_set_nvtx": (i32, [vp, i32]),
    "kxc_b200_plan_launch_info": (i32, [vp, i32, ctypes.c_char_p, i32, ctypes.POINTER(ctypes.c_double),
                                        ctypes.POINTER(ctypes.c_double)]),
    "kxc_b200_plan_run_timed": (i32, [vp, vpp, vp, ctypes.POINTER(ctypes.c_float), i32]),
}
_lib.SYMBOLS.update(_PLAN_SYMBOLS)


def _shape_arr(shape):
    return (i64 * max(len(shape), 1))(*[int(d) for d in shape])


def _attrs_c(call):
    a = call.attrs
    if call.op == "nn_conv2d":
        a = a or relay.Conv2DAttrs()
        pad = list(a.padding) + [0, 0]
        return Conv2dAttrsC((i32 * 2)(*a.strides[:2]), (i32 * 2)(pad[0], pad[1]), (i32 * 2)(*a.dilation[:2]), a.groups)
    if call.op == "nn_max_pool2d":
        pad = list(a.padding)
        if len(pad) == 2:
            pad = [pad[0], pad[1], pad[0], pad[1]]
        return Pool2dAttrsC((i32 * 2)(*a.pool_size[:2]), (i32 * 2)(*a.strides[:2]), (i32 * 4)(*pad[:4]), int(a.ceil_mode))
    if call.op == "nn_gemm":
        a = a or relay.GemmAttrs()
        return GemmAttrsC(a.alpha, a.beta, a.transA, a.transB)
    if call.op == "softmax":
        return SoftmaxAttrsC(int(a.axis) if a is not None else -1)
    if call.op == "nn_flatten" and a is not None:
        return FlattenAttrsC(int(a.axis))
    return None


class CompiledGraph:
    def __init__(self, func: relay.Function, precision="bf16", device=None, cuda_graph=False, nvtx=False):
        self.lib = load()
        self.func = func
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.handle = vp()
        check("plan_create", self.lib.kxc_b200_plan_create(PRECISIONS[precision], ctypes.byref(self.handle)))
        ids = {}

        def vid(e):
            if id(e) not in ids:
                ids[id(e)] = len(ids)
            return ids[id(e)]

        for p in func.params:
            check("plan_add_input", self.lib.kxc_b200_plan_add_input(self.handle, vid(p), len(p.shape), _shape_arr(p.shape)))
        self.constants = relay.constants_in_lowering_order(func)
        for c in self.constants:
            check("plan_add_constant",
                  self.lib.kxc_b200_plan_add_constant(self.handle, vid(c), len(c.shape), _shape_arr(c.shape)))
        for call in relay.post_order_calls(func):
            in_ids = (i32 * len(call.args))(*[vid(a) for a in call.args])
            attrs = _attrs_c(call)
            aptr = ctypes.cast(ctypes.pointer(attrs), vp) if attrs is not None else None
            check(f"plan_add_kernel({call.op})",
                  self.lib.kxc_b200_plan_add_kernel(self.handle, call.op.encode(), aptr, len(call.args), in_ids, vid(call)))
        out_id = vid(func.body)
        check("plan_set_output", self.lib.kxc_b200_plan_set_output(self.handle, out_id))
        with torch.cuda.device(self.device):
            check("plan_finalize", self.lib.kxc_b200_plan_finalize(self.handle))
        shp = (i64 * 6)()
        rank = self.lib.kxc_b200_plan_value_shape(self.handle, out_id, shp)
        self.out_shape = tuple(shp[i] for i in range(rank))
        self.num_launches = self.lib.kxc_b200_plan_num_launches(self.handle)
        if cuda_graph:
            check("plan_set_cuda_graph", self.lib.kxc_b200_plan_set_cuda_graph(self.handle, 1))
        if nvtx:
            self.set_nvtx(True)
        self.precision = precision
        self._const_ptrs = [c.data.data_ptr() for c in self.constants]
        for c in self.constants:
            assert c.data.is_cuda and c.data.dtype == torch.float32 and c.data.is_contiguous()

    def run(self, *inputs, out=None):
        """inputs: CUDA fp32 tensors in parameter order. Returns the output tensor (asynchronous)."""
        x = inputs[0]
        if out is None:
            out = torch.empty(self.out_shape, dtype=torch.float32, device=x.device)
        args = packed(*[t.data_ptr() for t in inputs], *self._const_ptrs, out.data_ptr())
        stream = torch.cuda.current_stream(x.device).cuda_stream
        check("kxc_kernel_main", self.lib.kxc_b200_plan_run(self.handle, args, stream))
        return out

    def set_nvtx(self, enable):
        """One NVTX range per run holding one range per launch (ProfileOptions::enable_nvtx of the reference)."""
        check("plan_set_nvtx", self.lib.kxc_b200_plan_set_nvtx(self.handle, 1 if enable else 0))

    def launch_info(self):
        """[(label, algorithmic flops, compulsory bytes)] per launch of one run."""
        out = []
        for i in range(self.num_launches):
            name = ctypes.create_string_buffer(192)
            fl, by = ctypes.c_double(0), ctypes.c_double(0)
            check("plan_launch_info", self.lib.kxc_b200_plan_launch_info(self.handle, i, name, 192, ctypes.byref(fl), ctypes.byref(by)))
            out.append((name.value.decode(), fl.value, by.value))
        return out

    def run_timed(self, *inputs, out=None):
        """One run with CUDA events between launches; returns (output, [ms per launch]). Synchronises."""
        x = inputs[0]
        if out is None:
            out = torch.empty(self.out_shape, dtype=torch.float32, device=x.device)
        args = packed(*[t.data_ptr() for t in inputs], *self._const_ptrs, out.data_ptr())
        ms = (ctypes.c_float * self.num_launches)()
        stream = torch.cuda.current_stream(x.device).cuda_stream
        check("plan_run_timed", self.lib.kxc_b200_plan_run_timed(self.handle, args, stream, ms, self.num_launches))
        return out, list(ms)

    def __del__(self):
        try:
            if self.handle:
                self.lib.kxc_b200_plan_destroy(self.handle)
                self.handle = None
        except Exception:
            pass

"""A minimal host-side mirror of the reference's Relay graph objects, enough to describe the graphs
its operator path runs: Var, Constant, Call, Function with the attribute structs the hot ops read.

It exists so that callers (tests, bench) build graphs the way the reference's own tests do
(test/op_numeric_llvm_test.cpp, test/resnet18_ir_dump.cpp) and so that the packed-argument order is
derived by the same rule the reference uses: function parameters, then constants in lowering DFS order
(arguments left to right, each expression visited once; test/onnx_importer_test.cpp:79-129,
src/relay/backend/lower.cc:534-565), then the output.
"""
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple


@dataclass(eq=False)
class Expr:
    pass


@dataclass(eq=False)
class Var(Expr):
    name: str
    shape: Tuple[int, ...]
    dtype: str = "float32"


@dataclass(eq=False)
class Constant(Expr):
    data: object  # a torch tensor (device) or numpy array; only shape is needed to build a plan
    name: str = ""

    @property
    def shape(self):
        return tuple(int(d) for d in self.data.shape)


@dataclass
class Conv2DAttrs:
    strides: Sequence[int] = (1, 1)
    padding: Sequence[int] = (0, 0, 0, 0)
    dilation: Sequence[int] = (1, 1)
    groups: int = 1


@dataclass
class MaxPool2DAttrs:
    strides: Sequence[int] = (1, 1)
    padding: Sequence[int] = (0, 0, 0, 0)
    dilation: Sequence[int] = (1, 1)
    pool_size: Sequence[int] = (1, 1)
    layout: str = "NCHW"
    ceil_mode: bool = False


@dataclass
class GemmAttrs:
    alpha: float = 1.0
    beta: float = 1.0
    transA: int = 0
    transB: int = 0


@dataclass
class SoftmaxAttrs:
    axis: int = -1


@dataclass
class FlattenAttrs:
    axis: int = 1  # FlattenAttrsNode (include/relay/op.h:353-358): dimensions before `axis` form the rows


@dataclass
class ReduceMeanAttrs:
    axis: Sequence[int] = ()
    keepdims: bool = True


@dataclass
class TransposeAttrs:
    axes: Sequence[int] = ()  # empty = reverse the dimensions


@dataclass
class ReshapeAttrs:
    newshape: Sequence[int] = ()
    allowzero: bool = False


@dataclass
class CastAttrs:
    dtype: str = "float32"  # the reference's dtype name


@dataclass(eq=False)
class Call(Expr):
    op: str  # Relay op name: "nn_conv2d", "nn_relu", "add", ...
    args: List[Expr] = field(default_factory=list)
    attrs: Optional[object] = None


@dataclass(eq=False)
class Function(Expr):
    params: List[Var]
    body: Expr


def post_order_calls(func: Function):
    """Calls in dependency order (DFS, arguments left to right, each expression once)."""
    seen, order = set(), []

    def visit(e):
        if id(e) in seen:
            return
        seen.add(id(e))
        if isinstance(e, Call):
            for a in e.args:
                visit(a)
            order.append(e)

    visit(func.body)
    return order


def constants_in_lowering_order(func: Function):
    seen, out = set(), []

    def visit(e):
        if id(e) in seen:
            return
        seen.add(id(e))
        if isinstance(e, Constant):
            out.append(e)
        elif isinstance(e, Call):
            for a in e.args:
                visit(a)

    visit(func.body)
    return out

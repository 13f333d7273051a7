"""Whole-graph CPU checker: walks a Relay-style function (hdkx_aicompiler_b200.relay objects) call by
call with the oracle's per-op functions, the way the reference lowers one loop nest per call
(src/relay/backend/lower.cc:567-617). TEST INFRASTRUCTURE ONLY.

`run(func, inputs)` is the reference arithmetic in fp32.

`run(func, inputs, operand_round=port.round_bf16)` is the same arithmetic with the roundings of a
reduced-precision mode applied where the GPU executor applies them: graph input and weights once,
and every activation the executor writes to memory (the value at the end of a fused
conv -> [add] -> [relu] chain, pooling outputs). The fusion rule is restated here independently:
a conv output with exactly one consumer that is an `add` (then one `nn_relu`) is not materialised.
"""
from concurrent.futures import ThreadPoolExecutor

import numpy as np

from . import port


def _consumers(calls):
    cons = {}
    for c in calls:
        for a in c.args:
            cons.setdefault(id(a), []).append(c)
    return cons


def _post_order(body):
    seen, order = set(), []

    def visit(e):
        if id(e) in seen:
            return
        seen.add(id(e))
        if hasattr(e, "args"):
            for a in e.args:
                visit(a)
            order.append(e)

    visit(body)
    return order


def _materialised(calls, body):
    """ids of call results that a fusing executor writes to memory. Calls are visited in dependency
    order; an add / relu can be absorbed by only one producer (the first that reaches it), so of the
    two convolutions feeding a residual add, the second one's result is materialised."""
    cons = _consumers(calls)
    fused_away, claimed = set(), set()

    def sole(c, op):
        cs = cons.get(id(c), [])
        return cs[0] if (len(cs) == 1 and cs[0].op == op and c is not body and id(cs[0]) not in claimed) else None

    for c in calls:
        if id(c) in claimed:
            continue
        if c.op == "nn_conv2d":
            cur = c
            a = sole(cur, "add")
            if a is not None:
                fused_away.add(id(cur))
                claimed.add(id(a))
                cur = a
            r = sole(cur, "nn_relu")
            if r is not None:
                fused_away.add(id(cur))
                claimed.add(id(r))
        elif c.op == "add":
            r = sole(c, "nn_relu")
            if r is not None:
                fused_away.add(id(c))
                claimed.add(id(r))
    return {id(c) for c in calls if id(c) not in fused_away}


def _batch_parallel(fn, x, workers):
    """Images are independent in every op: split dim 0 across threads (ctypes releases the GIL)."""
    n = x.shape[0]
    if workers <= 1 or n <= 1:
        return fn(x)
    parts = np.array_split(np.arange(n), min(workers, n))
    with ThreadPoolExecutor(len(parts)) as ex:
        outs = list(ex.map(lambda idx: fn(np.ascontiguousarray(x[idx[0]:idx[-1] + 1])), parts))
    return np.concatenate(outs, axis=0)


def run(func, inputs, operand_round=None, workers=1, backend=None):
    """backend: a module with the per-op functions (oracle.port by default, or oracle.ref for the
    reference compiler's own generated kernels)."""
    be = backend if backend is not None else port
    calls = _post_order(func.body)
    stored = _materialised(calls, func.body)
    rnd = operand_round if operand_round is not None else (lambda a: a)
    env = {}
    for p, x in zip(func.params, inputs):
        env[id(p)] = np.ascontiguousarray(x, dtype=np.float32)
    first_use_rounded = set()

    def val(e, as_operand=False):
        if id(e) in env:
            v = env[id(e)]
        else:  # Constant
            v = np.ascontiguousarray(np.asarray(e.data), dtype=np.float32)
        if as_operand and operand_round is not None and (id(e) not in first_use_rounded):
            # graph inputs and weights are rounded once when they enter a contraction
            if not hasattr(e, "args"):
                v = rnd(v)
        return v

    for c in calls:
        a = c.attrs
        if c.op == "nn_conv2d":
            x, w = val(c.args[0], True), val(c.args[1], True)
            b = val(c.args[2]) if len(c.args) == 3 else None
            s, p, d = tuple(a.strides[:2]), tuple(a.padding[:2]), tuple(a.dilation[:2])
            y = _batch_parallel(lambda xx: be.conv2d(xx, w, b, s, p, d), x, workers)
        elif c.op == "nn_relu":
            y = be.relu(val(c.args[0]))
        elif c.op == "add":
            y = be.add(val(c.args[0]), val(c.args[1]))
        elif c.op == "nn_max_pool2d":
            y = be.max_pool2d(val(c.args[0]), tuple(a.pool_size[:2]), tuple(a.strides[:2]), tuple(a.padding), a.ceil_mode)
        elif c.op == "nn_global_avg_pool2d":
            y = be.global_avg_pool2d(val(c.args[0]))
        elif c.op == "nn_flatten":
            v = val(c.args[0])
            axis = a.axis if a is not None else 1  # FlattenCompute (src/relay/op/tensor/transform.cc:140-182)
            axis = axis + v.ndim if axis < 0 else axis
            rows = 1
            for d in v.shape[:axis]:
                rows *= d
            y = v.reshape(rows, -1)
        elif c.op == "nn_dense":
            y = be.dense(val(c.args[0], True), val(c.args[1], True))
        elif c.op == "nn_gemm":
            y = be.gemm(val(c.args[0], True), val(c.args[1], True), val(c.args[2]), a.alpha, a.beta, a.transA, a.transB)
        elif c.op == "softmax":
            y = be.softmax(val(c.args[0]), a.axis if a is not None else -1)
        else:
            raise NotImplementedError(c.op)
        if operand_round is not None and id(c) in stored and c is not func.body:
            y = rnd(y)
        env[id(c)] = y
    return env[id(func.body)]

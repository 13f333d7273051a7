"""The reference's graph interchange format, "kxc.onnx_import.v1": a JSON description of a Relay function plus a
params.bin with the constants back to back (python/kxc_onnx/spec.py:61-103 writes it, LoadONNXImportSpec in
src/frontend/onnx_importer.cc:410-520 reads it). This module reads and writes the same files for the host-side graph
mirror in relay.py, so a graph exported by the reference's ONNX front end (or by save_spec below) can be handed to
plan.CompiledGraph, and a graph built here can be handed to the reference's importer.

Layout of the JSON (fields the reference's reader requires):
  format: "kxc.onnx_import.v1"
  function.inputs / function.outputs: [{name, shape, dtype}]
  function.nodes: [{name, op_name, inputs: [value names], outputs: [one value name], attrs: {...}}] in execution order
  params: [{name, shape, dtype, offset, nbytes}] (offsets into params.bin), param_order: [names]
Attribute keys per operator are the ones MakeAttrs reads (onnx_importer.cc:364-405): nn_conv2d {strides, pads,
dilations, group, channels, kernel_size, data_layout, kernel_layout, out_layout, out_dtype}; nn_max_pool2d {strides,
pads, dilations, pool_size, layout, ceil_mode}; nn_flatten {axis}; nn_gemm {alpha, beta, transA, transB}; nn_relu, add,
nn_global_avg_pool2d {}.
"""
import json

import numpy as np

from . import relay as R

FORMAT = "kxc.onnx_import.v1"
SUPPORTED = ("nn_conv2d", "nn_relu", "nn_max_pool2d", "add", "nn_global_avg_pool2d", "nn_flatten", "nn_gemm")


def _attrs_to_json(call):
    a = call.attrs
    if call.op == "nn_conv2d":
        w = call.args[1]
        return {"strides": list(a.strides), "pads": list(a.padding), "dilations": list(a.dilation), "group": int(a.groups),
                "channels": int(w.shape[0]), "kernel_size": [int(w.shape[2]), int(w.shape[3])], "data_layout": "NCHW",
                "kernel_layout": "OIHW", "out_layout": "", "out_dtype": ""}
    if call.op == "nn_max_pool2d":
        return {"strides": list(a.strides), "pads": list(a.padding), "dilations": list(a.dilation),
                "pool_size": list(a.pool_size), "layout": a.layout, "ceil_mode": bool(a.ceil_mode)}
    if call.op == "nn_flatten":
        return {"axis": int(a.axis) if a is not None else 1}
    if call.op == "nn_gemm":
        return {"alpha": float(a.alpha), "beta": float(a.beta), "transA": int(a.transA), "transB": int(a.transB)}
    return {}


def _attrs_from_json(op, d):
    if op == "nn_conv2d":
        return R.Conv2DAttrs(tuple(d["strides"]), tuple(d["pads"]), tuple(d["dilations"]), int(d["group"]))
    if op == "nn_max_pool2d":
        return R.MaxPool2DAttrs(tuple(d["strides"]), tuple(d["pads"]), tuple(d["dilations"]), tuple(d["pool_size"]),
                                d.get("layout", "NCHW"), bool(d["ceil_mode"]))
    if op == "nn_gemm":
        return R.GemmAttrs(float(d["alpha"]), float(d["beta"]), int(d["transA"]), int(d["transB"]))
    if op == "nn_flatten":  # the reference honours the axis (src/relay/op/tensor/transform.cc:145-165, type_infer.cc:446-450)
        return R.FlattenAttrs(int(d.get("axis", 1)))
    return None


def save_spec(func, out_shape, json_path, params_path):
    """Write `func` (constants as numpy arrays) in the reference's format. `out_shape` is the result's shape."""
    calls = R.post_order_calls(func)
    consts = R.constants_in_lowering_order(func)
    names = {}
    for v in func.params:
        names[id(v)] = v.name
    used = set(names.values())
    for i, c in enumerate(consts):
        n = c.name or f"param_{i}"
        while n in used:
            n += "_"
        used.add(n)
        names[id(c)] = n
    nodes = []
    for i, call in enumerate(calls):
        if call.op not in SUPPORTED:
            raise ValueError(f"operator {call.op} has no attribute encoding in {FORMAT}")
        names[id(call)] = f"v{i}"
        nodes.append({"name": f"{call.op}_{i}", "op_name": call.op, "inputs": [names[id(a)] for a in call.args],
                      "outputs": [f"v{i}"], "attrs": _attrs_to_json(call)})
    params, offset = [], 0
    with open(params_path, "wb") as f:
        for c in consts:
            arr = np.ascontiguousarray(np.asarray(c.data), dtype=np.float32)
            f.write(arr.tobytes())
            params.append({"name": names[id(c)], "shape": [int(d) for d in arr.shape], "dtype": "float32", "offset": offset,
                           "nbytes": int(arr.nbytes)})
            offset += int(arr.nbytes)
    spec = {
        "format": FORMAT,
        "function": {
            "inputs": [{"name": v.name, "shape": [int(d) for d in v.shape], "dtype": v.dtype} for v in func.params],
            "outputs": [{"name": names[id(func.body)], "shape": [int(d) for d in out_shape], "dtype": "float32"}],
            "nodes": nodes,
        },
        "params": params,
        "param_order": [p["name"] for p in params],
    }
    with open(json_path, "w", encoding="utf-8") as f:
        json.dump(spec, f, indent=2)
        f.write("\n")
    return spec


def load_spec(json_path, params_path, to_constant=None):
    """Read a graph in the reference's format into a relay.Function.

    `to_constant` converts each parameter (a numpy array) into what the Constants should hold, e.g. a CUDA tensor
    for plan.CompiledGraph; the default keeps numpy arrays. Returns (function, output shape). The same checks as the
    reference's reader: format tag, parameter byte ranges, param_order, one output per node, known value names.
    """
    with open(json_path, encoding="utf-8") as f:
        spec = json.load(f)
    if spec.get("format") != FORMAT:
        raise ValueError(f"Unsupported ONNX import spec format: {spec.get('format')}")
    blob = np.fromfile(params_path, dtype=np.uint8)
    values = {}
    params = []
    for v in spec["function"]["inputs"]:
        var = R.Var(v["name"], tuple(int(d) for d in v["shape"]), v["dtype"])
        params.append(var)
        values[v["name"]] = var
    order = []
    for p in spec["params"]:
        off, nb = int(p["offset"]), int(p["nbytes"])
        if off < 0 or nb < 0 or off + nb > blob.size:
            raise ValueError(f"Param bytes range out of bounds for: {p['name']}")
        if p["dtype"] != "float32":
            raise ValueError(f"parameter {p['name']}: dtype {p['dtype']} is not supported")
        arr = blob[off:off + nb].view(np.float32).reshape([int(d) for d in p["shape"]]).copy()
        values[p["name"]] = R.Constant(to_constant(arr) if to_constant else arr, p["name"])
        order.append(p["name"])
    if "param_order" in spec and list(spec["param_order"]) != order:
        raise ValueError("ONNX import spec param_order does not match params metadata")
    for node in spec["function"]["nodes"]:
        if len(node["outputs"]) != 1:
            raise ValueError(f"ONNX import node must have one output: {node['name']}")
        args = []
        for name in node["inputs"]:
            if name not in values:
                raise ValueError(f"Missing input value '{name}' for node '{node['name']}'")
            args.append(values[name])
        op = node["op_name"]
        if op not in SUPPORTED:
            raise ValueError(f"Unsupported Relay op in ONNX import spec: {op}")
        values[node["outputs"][0]] = R.Call(op, args, _attrs_from_json(op, node.get("attrs", {})))
    outs = spec["function"]["outputs"]
    if len(outs) != 1:
        raise ValueError("exactly one graph output is supported")
    if outs[0]["name"] not in values:
        raise ValueError(f"Missing graph output value in ONNX import spec: {outs[0]['name']}")
    return R.Function(params, values[outs[0]["name"]]), tuple(int(d) for d in outs[0]["shape"])

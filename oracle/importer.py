"""The reference's own graph importer as a checker. TEST INFRASTRUCTURE ONLY.

`describe(json, params)` runs oracle/_ref/ref_emit --import, i.e. the UNMODIFIED LoadONNXImportSpec
(src/frontend/onnx_importer.cc:410-520) followed by the reference's InferTypePass, and returns the Relay function it
built: inputs, calls in post order with the attribute values its Attrs objects hold and the shapes it inferred, and the
result. `to_relay` turns that description into hdkx_aicompiler_b200.relay objects, so a test can run exactly the graph
the reference's importer built through the CPU oracle and through the GPU executor, and can compare it with the graph
the package's own reader (hdkx_aicompiler_b200/onnx_import.py) builds from the same files.
"""
import json
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_EMIT = os.path.join(_HERE, "_ref", "ref_emit")


def available():
    return os.path.exists(_EMIT)


def describe(json_path, params_path):
    out = subprocess.run([_EMIT, "--import", json_path, params_path], check=True, capture_output=True, text=True).stdout
    return json.loads(out)


def read_params(json_path, params_path):
    """name -> numpy array, from the spec's parameter table."""
    with open(json_path, encoding="utf-8") as f:
        spec = json.load(f)
    blob = np.fromfile(params_path, dtype=np.uint8)
    return {p["name"]: blob[p["offset"]:p["offset"] + p["nbytes"]].view(np.float32).reshape(p["shape"]).copy()
            for p in spec["params"]}


def to_relay(desc, params, to_constant=None):
    """Build relay objects from `describe`'s output. Returns (function, output shape)."""
    from hdkx_aicompiler_b200 import relay as R

    inputs = {v["name"]: R.Var(v["name"], tuple(v["shape"]), v["dtype"]) for v in desc["inputs"]}
    consts, nodes = {}, {}

    def ref(a):
        if "var" in a:
            return inputs[a["var"]]
        if "param" in a:
            name = a["param"]
            if name not in consts:
                arr = params[name]
                consts[name] = R.Constant(to_constant(arr) if to_constant else arr, name)
            return consts[name]
        return nodes[a["node"]]

    shape = None
    for n in desc["nodes"]:
        at, op = n["attrs"], n["op"]
        attrs = None
        if op == "nn_conv2d":
            attrs = R.Conv2DAttrs(tuple(at["strides"]), tuple(at["padding"]), tuple(at["dilation"]), at["groups"])
        elif op in ("nn_max_pool2d", "nn_avg_pool2d"):
            attrs = R.MaxPool2DAttrs(tuple(at["strides"]), tuple(at["padding"]), tuple(at["dilation"]), tuple(at["pool_size"]),
                                     "NCHW", bool(at["ceil_mode"]))
        elif op == "nn_gemm":
            attrs = R.GemmAttrs(at["alpha"], at["beta"], at["transA"], at["transB"])
        elif op == "nn_flatten":
            attrs = R.FlattenAttrs(int(at.get("axis", 1)))
        nodes[n["id"]] = R.Call(op, [ref(a) for a in n["args"]], attrs)
        shape = tuple(n["shape"])
    body = ref(desc["result"])
    if "node" in desc["result"]:
        shape = tuple(next(n["shape"] for n in desc["nodes"] if n["id"] == desc["result"]["node"]))
    return R.Function([inputs[v["name"]] for v in desc["inputs"]], body), shape

"""The reference's graph interchange format ("kxc.onnx_import.v1") as a feed for both executors: a graph written by
hdkx_aicompiler_b200.onnx_import.save_spec is read back (a) by the package's own reader and (b) by the reference's
UNMODIFIED importer (oracle/_ref/ref_emit --import); both must build the same calls, attributes and shapes, and the
CPU oracle must produce the same bits from either. A committed fixture pins the format and one output."""
import json
import os

import numpy as np
import pytest

from hdkx_aicompiler_b200 import onnx_import, relay as R, resnet18
from oracle import graph as ograph
from oracle import importer as oimp

f32 = np.float32
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
needs_ref = pytest.mark.skipif(not oimp.available(), reason="oracle/_ref/ref_emit is not built")


def small_block(rng):
    """A residual downsample block with a stem-like front: every operator the format encodes."""
    x = R.Var("input", (2, 3, 20, 20))
    k = lambda *s: rng.normal(0, 0.2, s).astype(f32)  # noqa: E731
    conv = lambda d, w, b, s, p: R.Call("nn_conv2d", [d, R.Constant(w), R.Constant(b)],  # noqa: E731
                                        R.Conv2DAttrs((s, s), (p, p, p, p), (1, 1), 1))
    y = R.Call("nn_relu", [conv(x, k(8, 3, 3, 3), k(8), 2, 1)])
    y = R.Call("nn_max_pool2d", [y], R.MaxPool2DAttrs((2, 2), (1, 1, 1, 1), (1, 1), (3, 3), "NCHW", False))
    a = R.Call("nn_relu", [conv(y, k(16, 8, 3, 3), k(16), 2, 1)])
    a = conv(a, k(16, 16, 3, 3), k(16), 1, 1)
    d = conv(y, k(16, 8, 1, 1), k(16), 2, 0)
    z = R.Call("nn_relu", [R.Call("add", [a, d])])
    z = R.Call("nn_flatten", [R.Call("nn_global_avg_pool2d", [z])])
    out = R.Call("nn_gemm", [z, R.Constant(k(10, 16)), R.Constant(k(10))], R.GemmAttrs(1.0, 1.0, 0, 1))
    return R.Function([x], out), (2, 10)


def signature(func):
    """Operators, attribute values and argument wiring of a function, independent of object identity."""
    calls = R.post_order_calls(func)
    index = {id(c): i for i, c in enumerate(calls)}
    sig = []
    for c in calls:
        args = []
        for a in c.args:
            if isinstance(a, R.Call):
                args.append(("node", index[id(a)]))
            elif isinstance(a, R.Constant):
                args.append(("param", a.name, tuple(a.shape)))
            else:
                args.append(("var", a.name, tuple(a.shape)))
        at = c.attrs
        if at is None:
            attrs = ()
        else:
            attrs = tuple((k, tuple(v) if isinstance(v, (list, tuple)) else v) for k, v in sorted(vars(at).items()) if k != "layout")
        sig.append((c.op, tuple(args), attrs))
    return sig


def test_roundtrip_through_own_reader(tmp_path, rng):
    func, out_shape = small_block(rng)
    j, p = str(tmp_path / "g.json"), str(tmp_path / "g.bin")
    onnx_import.save_spec(func, out_shape, j, p)
    back, shape = onnx_import.load_spec(j, p)
    assert shape == out_shape
    # parameter names are assigned by save_spec: compare wiring and values
    named = onnx_import.load_spec(j, p)[0]
    assert [s[0] for s in signature(back)] == [s[0] for s in signature(func)]
    x = rng.normal(0, 1, (2, 3, 20, 20)).astype(f32)
    a, b = ograph.run(func, [x]), ograph.run(named, [x])
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_reader_rejects_what_the_reference_rejects(tmp_path, rng):
    func, out_shape = small_block(rng)
    j, p = str(tmp_path / "g.json"), str(tmp_path / "g.bin")
    spec = onnx_import.save_spec(func, out_shape, j, p)
    bad = dict(spec, format="kxc.onnx_import.v0")
    (tmp_path / "bad.json").write_text(json.dumps(bad))
    with pytest.raises(ValueError, match="Unsupported ONNX import spec format"):
        onnx_import.load_spec(str(tmp_path / "bad.json"), p)
    bad = json.loads(json.dumps(spec))
    bad["params"][0]["nbytes"] = 10 ** 9
    (tmp_path / "bad.json").write_text(json.dumps(bad))
    with pytest.raises(ValueError, match="out of bounds"):
        onnx_import.load_spec(str(tmp_path / "bad.json"), p)
    bad = json.loads(json.dumps(spec))
    bad["function"]["nodes"][0]["inputs"][0] = "nowhere"
    (tmp_path / "bad.json").write_text(json.dumps(bad))
    with pytest.raises(ValueError, match="Missing input value"):
        onnx_import.load_spec(str(tmp_path / "bad.json"), p)


@needs_ref
@pytest.mark.parametrize("which", ["block", "resnet18"])
def test_reference_importer_builds_the_same_graph(tmp_path, rng, which):
    if which == "block":
        func, out_shape = small_block(rng)
        x = rng.normal(0, 1, (2, 3, 20, 20)).astype(f32)
    else:
        func, out_shape = resnet18.build(1, resnet18.make_weights(seed=0)), (1, 1000)
        x = rng.normal(0, 1, (1, 3, 224, 224)).astype(f32)
    j, p = str(tmp_path / "g.json"), str(tmp_path / "g.bin")
    onnx_import.save_spec(func, out_shape, j, p)
    desc = oimp.describe(j, p)                       # the reference's importer + InferTypePass
    ref_func, ref_shape = oimp.to_relay(desc, oimp.read_params(j, p))
    own_func, own_shape = onnx_import.load_spec(j, p)
    assert ref_shape == own_shape == out_shape       # the reference's inferred result shape
    assert signature(ref_func) == signature(own_func)
    got = ograph.run(ref_func, [x], workers=4)
    exp = ograph.run(func, [x], workers=4)
    assert np.array_equal(got.view(np.uint32), exp.view(np.uint32))


def test_committed_fixture():
    """tests/golden/import_block.{json,bin}: written by save_spec, read back by the reference's importer and run
    through the reference-built CPU kernels by tests/golden/make_import_fixture.py; the expected output is committed."""
    j, p = os.path.join(GOLDEN, "import_block.json"), os.path.join(GOLDEN, "import_block.bin")
    ref = np.load(os.path.join(GOLDEN, "import_block_io.npz"))
    func, shape = onnx_import.load_spec(j, p)
    assert shape == tuple(ref["output"].shape)
    got = ograph.run(func, [ref["input"]])
    assert np.array_equal(got.view(np.uint32), ref["output"].view(np.uint32))


@needs_ref
def test_flatten_axis_is_carried_and_agrees_with_the_reference(tmp_path, rng):
    """nn_flatten's axis survives the loader (the reference honours it: src/relay/op/tensor/transform.cc:145-165,
    src/relay/type_infer.cc:446-450): for axis 2 both readers see the attribute and the reference's inferred result shape is
    the one the CPU checker produces."""
    w = rng.normal(0, 0.2, (4, 3, 3, 3)).astype(f32)
    x = R.Var("input", (2, 3, 8, 8))
    y = R.Call("nn_relu", [R.Call("nn_conv2d", [x, R.Constant(w, "w")], R.Conv2DAttrs((1, 1), (1, 1, 1, 1), (1, 1), 1))])
    func = R.Function([x], R.Call("nn_flatten", [y], R.FlattenAttrs(2)))
    j, p = str(tmp_path / "f.json"), str(tmp_path / "f.bin")
    onnx_import.save_spec(func, (8, 64), j, p)
    own, own_shape = onnx_import.load_spec(j, p)
    assert R.post_order_calls(own)[-1].attrs == R.FlattenAttrs(2)
    desc = oimp.describe(j, p)                       # the reference's importer + InferTypePass
    ref_func, ref_shape = oimp.to_relay(desc, oimp.read_params(j, p))
    assert ref_shape == own_shape == (8, 64)
    assert signature(ref_func) == signature(own)
    xin = rng.normal(0, 1, (2, 3, 8, 8)).astype(f32)
    assert ograph.run(own, [xin]).shape == (8, 64)


@pytest.mark.gpu
def test_plan_refuses_flatten_at_another_axis(rng):
    """A plan flattens at axis 1 (negative values normalised) and refuses anything else instead of silently producing a
    shape the reference would not."""
    import torch
    from hdkx_aicompiler_b200 import KxcError, plan
    w = torch.from_numpy(rng.normal(0, 0.2, (16, 16, 3, 3)).astype(f32)).cuda()

    def build(axis):
        x = R.Var("input", (2, 16, 8, 8))
        y = R.Call("nn_relu", [R.Call("nn_conv2d", [x, R.Constant(w, "w")], R.Conv2DAttrs((1, 1), (1, 1, 1, 1), (1, 1), 1))])
        y = R.Call("nn_global_avg_pool2d", [y])
        return R.Function([x], R.Call("nn_relu", [R.Call("nn_flatten", [y], R.FlattenAttrs(axis))]))

    for ok_axis in (1, -3):
        g = plan.CompiledGraph(build(ok_axis), "fp32")
        assert g.out_shape == (2, 16)
    with pytest.raises(KxcError, match="axis"):
        plan.CompiledGraph(build(2), "fp32")

"""The reference's ExecutionPlan JSON as a feed: tests/golden/import_block_plan.json is what the reference's own
LowerRelayToExecPlanPass + SerializeExecutionPlanToJson produced for the graph of tests/golden/import_block.*. The
package reads it, names a kernel for every KernelExec node, and executes it node by node (per-operator C ABI) or as one
compiled graph; the fp32 results must be the bits the reference's generated CPU kernels gave for the same graph."""
import json
import os
import subprocess

import numpy as np
import pytest

from hdkx_aicompiler_b200 import execution_plan as xp
from hdkx_aicompiler_b200 import onnx_import
from test_onnx_import import signature

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
EMIT = os.path.join(os.path.dirname(GOLDEN), "..", "oracle", "_ref", "ref_emit")
needs_ref = pytest.mark.skipif(not os.path.exists(EMIT), reason="oracle/_ref/ref_emit is not built")


def fixture():
    plan = xp.load(open(os.path.join(GOLDEN, "import_block_plan.json")).read())
    spec = json.load(open(os.path.join(GOLDEN, "import_block.json")))
    return plan, spec


def constants_of(plan, to_constant=None):
    """The spec's parameters in constant_value_ids order (both follow the function's DFS order)."""
    func, _ = onnx_import.load_spec(os.path.join(GOLDEN, "import_block.json"), os.path.join(GOLDEN, "import_block.bin"), to_constant)
    from hdkx_aicompiler_b200 import relay as R
    consts = [c.data for c in R.constants_in_lowering_order(func)]
    shapes = xp._shapes(plan)
    assert [tuple(c.shape) for c in consts] == [shapes[i] for i in plan["constant_value_ids"]]
    return consts, func


def test_plan_fixture_structure_and_symbols():
    plan, spec = fixture()
    nodes = xp.kernel_nodes(plan)
    assert [n["op_name"] for n in nodes] == [n["op_name"] for n in spec["function"]["nodes"]]
    assert all(n["kernel_symbol"] == "" and n["worker_set"] == [0] for n in nodes)  # reserved and empty in the reference
    bound = xp.bind_kernel_symbols(plan)
    import hdkx_aicompiler_b200 as kxc
    lib = kxc.load()
    for n in xp.kernel_nodes(bound):
        assert n["kernel_symbol"] == xp.KERNEL_SYMBOLS[n["op_name"]] and hasattr(lib, n["kernel_symbol"])
    assert xp.kernel_nodes(plan)[0]["kernel_symbol"] == ""  # the input is not modified
    assert xp.load(xp.dumps(bound)) == bound
    attrs = xp.attrs_from_import_spec(plan, spec)
    consts, func = constants_of(plan)
    rebuilt = xp.to_function(plan, attrs, consts)
    assert [(s[0], s[2]) for s in signature(rebuilt)] == [(s[0], s[2]) for s in signature(func)]
    wiring = lambda f: [tuple(a[0] if a[0] != "node" else a for a in s[1]) for s in signature(f)]  # noqa: E731
    assert wiring(rebuilt) == wiring(func)
    with pytest.raises(ValueError, match="schema_version"):
        xp.load(json.dumps(dict(plan, schema_version=2)))
    with pytest.raises(ValueError, match="kernel nodes"):
        xp.attrs_from_import_spec(dict(plan, nodes=plan["nodes"][:-1]), spec)


@needs_ref
def test_reference_builds_this_plan_and_reads_the_bound_one(tmp_path):
    """The committed fixture is what the reference emits today, and the reference's reader accepts the plan with the
    kernel symbols filled in and serializes it back unchanged."""
    out = subprocess.run([EMIT, "--plan", os.path.join(GOLDEN, "import_block.json"), os.path.join(GOLDEN, "import_block.bin")],
                         check=True, capture_output=True, text=True).stdout
    assert out == open(os.path.join(GOLDEN, "import_block_plan.json")).read()
    plan, _ = fixture()
    bound = xp.bind_kernel_symbols(plan)
    path = tmp_path / "bound.json"
    path.write_text(xp.dumps(bound))
    back = subprocess.run([EMIT, "--plan-check", str(path)], check=True, capture_output=True, text=True).stdout
    assert xp.load(back) == bound


@pytest.mark.gpu
def test_execute_plan_on_gpu():
    import torch
    from conftest import assert_bit_exact, assert_close
    from hdkx_aicompiler_b200 import ops, plan as kplan
    to_cuda = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()  # noqa: E731
    p, spec = fixture()
    attrs = xp.attrs_from_import_spec(p, spec)
    consts, _ = constants_of(p, to_cuda)
    io = np.load(os.path.join(GOLDEN, "import_block_io.npz"))
    x = to_cuda(io["input"])
    # node by node through the per-operator entry points, fp32 kernels in the reference's order: the reference's bits
    got = xp.execute_kernels(p, attrs, consts, [x], precision="fp32").cpu().numpy()
    assert_bit_exact(got, io["output"], "ExecutionPlan interpreted node by node, fp32")
    got3 = xp.execute_kernels(p, attrs, consts, [x], precision="tf32x3").cpu().numpy()
    assert_close(got3, io["output"], 1e-4, "ExecutionPlan interpreted node by node, three-pass tf32")
    # the same plan as one compiled graph
    g = kplan.CompiledGraph(xp.to_function(p, attrs, consts), "fp32")
    assert_bit_exact(g.run(x).cpu().numpy(), io["output"], "ExecutionPlan as one compiled graph, fp32")
    assert ops.device_status() == 0


def test_null_nodes_are_skipped_like_the_reference_does():
    """The reference's writer emits `null` for an undefined node and its reader skips it (src/base/execution_plan.cc:689-692)."""
    text = open(os.path.join(GOLDEN, "import_block_plan.json")).read()
    plan = json.loads(text)
    n = len(plan["nodes"])
    plan["nodes"].insert(1, None)
    plan["nodes"].append(None)
    loaded = xp.load(json.dumps(plan))
    assert len(loaded["nodes"]) == n and all(node is not None for node in loaded["nodes"])
    assert len(xp.kernel_nodes(loaded)) == len(xp.kernel_nodes(xp.load(text)))
    assert xp.bind_kernel_symbols(loaded) == xp.bind_kernel_symbols(xp.load(text))


@pytest.mark.gpu
def test_every_bound_operator_executes():
    """Every operator bind_kernel_symbols accepts is one execute_kernels can run: the five outside the ResNet path too."""
    import torch
    from conftest import assert_bit_exact
    from hdkx_aicompiler_b200 import relay as R
    from oracle import port
    rng = np.random.default_rng(9)
    x = rng.normal(0, 1, (2, 4, 6, 6)).astype(np.float32)
    nodes = [
        ("nn_avg_pool2d", R.MaxPool2DAttrs((2, 2), (0, 0, 0, 0), (1, 1), (2, 2), "NCHW", False)),
        ("reduce_mean", R.ReduceMeanAttrs((2, 3), True)),
        ("transpose", R.TransposeAttrs((1, 0, 2, 3))),
        ("reshape", R.ReshapeAttrs((4, 2), False)),
        ("cast", R.CastAttrs("int32")),
    ]
    plan = {"schema_version": 1, "num_values": 6, "output_value": 5, "input_value_ids": [0], "constant_value_ids": [],
            "value_info": [{"value_id": 0, "shape": list(x.shape), "dtype": "float32"}],
            "nodes": [{"kind": "kernel", "op_name": op, "kernel_symbol": "", "input_values": [i], "output_values": [i + 1], "worker_set": []}
                      for i, (op, _) in enumerate(nodes)]}
    bound = xp.bind_kernel_symbols(xp.load(json.dumps(plan)))
    assert [n["kernel_symbol"] for n in bound["nodes"]] == ["kxc_b200_nn_avg_pool2d", "kxc_b200_reduce_mean", "kxc_b200_transpose",
                                                            "kxc_b200_reshape", "kxc_b200_cast"]
    got = xp.execute_kernels(bound, [a for _, a in nodes], [], [torch.from_numpy(x).cuda()]).cpu().numpy()
    exp = port.avg_pool2d(x, (2, 2), (2, 2), (0, 0, 0, 0))
    exp = port.reduce_mean(exp, (2, 3), True)
    exp = np.ascontiguousarray(exp.transpose(1, 0, 2, 3)).reshape(4, 2).astype(np.int32)
    assert got.dtype == np.int32 and got.shape == (4, 2)
    assert np.array_equal(got, exp)

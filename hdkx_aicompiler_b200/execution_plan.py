"""The reference's runtime ExecutionPlan, read from its own JSON form and executed on this library.

The reference lowers a Relay function to an ExecutionPlan (LowerRelayToExecPlanPass,
src/relay/transforms/multi_device.cc:244-) whose KernelExec nodes carry {op_name, kernel_symbol (reserved, empty today),
input_values, output_values, worker_set} (include/base/execution_plan.h:42-50) and serializes it with
SerializeExecutionPlanToJson (src/base/execution_plan.cc:672-772). Its executor runs every KernelExec node as a placeholder
copy (src/base/disco/executor.cc:122-157). This module is what stands behind those nodes here:

  load / dumps            the JSON as the reference writes it (schema_version 1), unchanged on the way out
  bind_kernel_symbols     fills each KernelExec node's reserved `kernel_symbol` with the C-ABI entry point that runs it
  attrs_from_import_spec  the attribute side table (the plan JSON drops operator attributes, execution_plan.cc:695-708):
                          one entry per KernelExec node, taken from the "kxc.onnx_import.v1" spec the plan was built from
  execute_kernels         the KernelExec interpreter: one kxc_b200_<op> call per node, values held by id like the
                          reference's register file
  to_function             the same plan as a relay.Function for plan.CompiledGraph (the whole-graph entry point)

Comm and barrier nodes: a barrier is a stream-ordered no-op on one worker; `device.gather_to_worker0` is
parallel.GatherToWorker0 / PeerStoreToWorker0. Plans with other communication nodes are refused.
"""
import json

from . import ops, relay as R

SCHEMA_VERSION = 1

# KernelExec op_name -> the entry point of include/kxc_b200.h that executes it
KERNEL_SYMBOLS = {
    "nn_conv2d": "kxc_b200_nn_conv2d", "nn_relu": "kxc_b200_nn_relu", "add": "kxc_b200_add",
    "nn_max_pool2d": "kxc_b200_nn_max_pool2d", "nn_avg_pool2d": "kxc_b200_nn_avg_pool2d",
    "nn_global_avg_pool2d": "kxc_b200_nn_global_avg_pool2d", "nn_flatten": "kxc_b200_nn_flatten",
    "nn_dense": "kxc_b200_nn_gemm", "nn_gemm": "kxc_b200_nn_gemm", "softmax": "kxc_b200_softmax",
    "reduce_mean": "kxc_b200_reduce_mean", "matmul": "kxc_b200_matmul", "transpose": "kxc_b200_transpose",
    "reshape": "kxc_b200_reshape", "cast": "kxc_b200_cast",
}


def load(text):
    """Parse an ExecutionPlan JSON; the same checks as DeserializeExecutionPlanFromJson makes first."""
    plan = json.loads(text)
    if not isinstance(plan, dict):
        raise ValueError("ExecutionPlan JSON root must be an object")
    if plan.get("schema_version") != SCHEMA_VERSION:
        raise ValueError(f"Unsupported ExecutionPlan JSON schema_version: {plan.get('schema_version')}")
    for key in ("num_values", "output_value", "nodes", "input_value_ids", "constant_value_ids", "value_info"):
        if key not in plan:
            raise ValueError(f"ExecutionPlan JSON is missing '{key}'")
    # the reference's writer emits `null` for an undefined node and its reader skips such entries
    # (src/base/execution_plan.cc:689-692): they are dropped here
    plan["nodes"] = [n for n in plan["nodes"] if n is not None]
    for i, node in enumerate(plan["nodes"]):
        if not isinstance(node, dict) or node.get("kind") not in ("kernel", "comm", "barrier"):
            raise ValueError(f"ExecutionPlan JSON node {i} has unknown kind: {node.get('kind') if isinstance(node, dict) else node}")
    return plan


def dumps(plan):
    """Compact JSON with the reference's key order preserved (json keeps insertion order)."""
    return json.dumps(plan, separators=(",", ":"))


def kernel_nodes(plan):
    return [n for n in plan["nodes"] if n["kind"] == "kernel"]


def bind_kernel_symbols(plan):
    """A copy of the plan whose KernelExec nodes name the entry point that executes them."""
    out = json.loads(json.dumps(plan))
    for node in kernel_nodes(out):
        if node["op_name"] not in KERNEL_SYMBOLS:
            raise ValueError(f"no kernel for op '{node['op_name']}'")
        node["kernel_symbol"] = KERNEL_SYMBOLS[node["op_name"]]
    return out


def attrs_from_import_spec(plan, spec):
    """Attribute side table: relay attrs objects, one per KernelExec node, in node order. Both the plan builder and the
    import spec list the calls in execution (post-DFS) order; operator names are cross-checked."""
    from .onnx_import import _attrs_from_json
    nodes, spec_nodes = kernel_nodes(plan), spec["function"]["nodes"]
    if len(nodes) != len(spec_nodes):
        raise ValueError(f"plan has {len(nodes)} kernel nodes, the import spec {len(spec_nodes)}")
    table = []
    for i, (pn, sn) in enumerate(zip(nodes, spec_nodes)):
        if pn["op_name"] != sn["op_name"]:
            raise ValueError(f"node {i}: plan runs '{pn['op_name']}', the import spec '{sn['op_name']}'")
        table.append(_attrs_from_json(sn["op_name"], sn.get("attrs", {})))
    return table


def _shapes(plan):
    return {int(v["value_id"]): tuple(int(d) for d in v["shape"]) for v in plan["value_info"]}


def to_function(plan, attrs, constants):
    """relay.Function equivalent to the plan. `constants`: one array / tensor per entry of constant_value_ids, in that
    order (the order of the packed constant arguments)."""
    if len(constants) != len(plan["constant_value_ids"]):
        raise ValueError("one constant per constant_value_id is required")
    shapes = _shapes(plan)
    values, params = {}, []
    for k, vid in enumerate(plan["input_value_ids"]):
        var = R.Var(f"input{k}" if k else "input", shapes[vid], "float32")
        values[vid] = var
        params.append(var)
    for vid, data in zip(plan["constant_value_ids"], constants):
        values[vid] = R.Constant(data, f"v{vid}")
    k = 0
    for node in plan["nodes"]:
        if node["kind"] == "barrier":
            continue
        if node["kind"] != "kernel":
            raise NotImplementedError(f"communication node '{node.get('op_name')}' inside a single-worker function")
        if len(node["output_values"]) != 1:
            raise ValueError("a KernelExec node must have one output value")
        values[node["output_values"][0]] = R.Call(node["op_name"], [values[i] for i in node["input_values"]], attrs[k])
        k += 1
    return R.Function(params, values[plan["output_value"]])


def _run_kernel(op, a, args, precision):
    if op == "nn_conv2d":
        a = a or R.Conv2DAttrs()
        return ops.nn_conv2d(args[0], args[1], args[2] if len(args) > 2 else None, tuple(a.strides[:2]), tuple(a.padding[:2]),
                             tuple(a.dilation[:2]), a.groups, precision=precision)
    if op == "nn_relu":
        return ops.nn_relu(args[0])
    if op == "add":
        return ops.add(args[0], args[1])
    if op == "nn_max_pool2d":
        return ops.nn_max_pool2d(args[0], tuple(a.pool_size[:2]), tuple(a.strides[:2]), tuple(a.padding), a.ceil_mode)
    if op == "nn_global_avg_pool2d":
        return ops.nn_global_avg_pool2d(args[0])
    if op == "nn_flatten":
        return ops.nn_flatten(args[0])
    if op == "nn_dense":
        return ops.nn_dense(args[0], args[1], precision=precision)
    if op == "nn_gemm":
        a = a or R.GemmAttrs()
        return ops.nn_gemm(args[0], args[1], args[2], a.alpha, a.beta, a.transA, a.transB, precision=precision)
    if op == "softmax":
        return ops.softmax(args[0], a.axis if a is not None else -1)
    if op == "matmul":
        return ops.matmul(args[0], args[1], precision=precision)
    if op == "nn_avg_pool2d":
        return ops.nn_avg_pool2d(args[0], tuple(a.pool_size[:2]), tuple(a.strides[:2]), tuple(a.padding), a.ceil_mode)
    if op == "reduce_mean":
        return ops.reduce_mean(args[0], tuple(a.axis), bool(a.keepdims))
    if op == "transpose":
        return ops.transpose(args[0], tuple(a.axes) if a is not None and a.axes else None)
    if op == "reshape":
        return ops.reshape(args[0], tuple(a.newshape), bool(a.allowzero))
    if op == "cast":
        return ops.cast(args[0], a.dtype)
    raise NotImplementedError(f"no kernel for op '{op}'")


def execute_kernels(plan, attrs, constants, inputs, precision="fp32"):
    """Interpret the plan node by node: every KernelExec node is one call of the per-operator C ABI on CUDA tensors.
    Returns the tensor of plan['output_value']. Values no later node reads are dropped as the walk passes them."""
    values = {}
    for vid, t in zip(plan["input_value_ids"], inputs):
        values[vid] = t
    for vid, t in zip(plan["constant_value_ids"], constants):
        values[vid] = t
    last_use = {}
    for idx, node in enumerate(plan["nodes"]):
        for i in node.get("input_values", []):
            last_use[i] = idx
    k = 0
    for idx, node in enumerate(plan["nodes"]):
        if node["kind"] == "barrier":
            continue  # one worker, one stream: launches are already ordered
        if node["kind"] != "kernel":
            raise NotImplementedError(f"communication node '{node.get('op_name')}': use parallel.GatherToWorker0")
        args = [values[i] for i in node["input_values"]]
        values[node["output_values"][0]] = _run_kernel(node["op_name"], attrs[k], args, precision)
        k += 1
        for i in node["input_values"]:
            if last_use.get(i) == idx and i != plan["output_value"] and i not in plan["constant_value_ids"]:
                values.pop(i, None)
    return values[plan["output_value"]]

"""Profiling integration: events in the reference's bundle format (CPU), NVTX ranges and a profiled run (GPU)."""
import json
import os
import subprocess
import sys

import pytest

from hdkx_aicompiler_b200 import profiling
from profile_cases import CASES, build_case

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)

# what the reference's reader requires of every event (python/kxc_agent/services/schema.py:11-32)
REQUIRED = ("trace_id", "session_id", "run_id", "span_id", "parent_span_id", "component", "event_type", "phase", "ts_ns",
            "duration_ns", "status", "severity", "device", "worker_id", "op_name", "pass_name", "kernel_symbol",
            "shape_signature", "message", "metrics")
BUNDLE_FILES = ("manifest.json", "events.jsonl", "trace.json", "summary.json", "diagnosis.json", "diagnosis.md")


def _rules(events):
    """The two device-side rules of the reference's agent (python/kxc_agent/services/diagnosis_engine.py:236-300,
    thresholds from rule_library.py): copy share of device_api time >= 0.40; >= 5 module runs shorter than 200 us."""
    found = []
    dev = sum(e["duration_ns"] for e in events if e["component"] == "device_api")
    cp = sum(e["duration_ns"] for e in events if e["component"] == "device_api" and e["event_type"] == "copy")
    if dev > 0 and cp / dev >= 0.40:
        found.append("copy_dominance")
    tiny = [e for e in events if e["event_type"] in ("compiled_module_run", "adaptive_module_run") and e["duration_ns"] < 200_000]
    if len(tiny) >= 5:
        found.append("kernel_launch_overhead")
    return found


@pytest.mark.parametrize("case", CASES)
def test_bundle_matches_what_the_reference_agent_accepted(case, tmp_path):
    b = build_case(case, str(tmp_path))
    b.write()
    for name in BUNDLE_FILES:
        assert (tmp_path / name).exists(), name
    assert (tmp_path / "artifacts").is_dir()
    events = [json.loads(line) for line in open(tmp_path / "events.jsonl")]
    assert events and len(events) == len(b.events)
    for ev in events:
        assert tuple(ev) == profiling.EVENT_KEYS
        assert all(k in ev for k in REQUIRED)
        assert isinstance(ev["ts_ns"], int) and isinstance(ev["duration_ns"], int) and ev["duration_ns"] >= 0
        assert ev["fields"]["schema_version"] == "1"
    assert json.load(open(tmp_path / "manifest.json"))["schema_version"] == 1
    assert json.load(open(tmp_path / "summary.json"))["event_count"] == len(events)
    trace = json.load(open(tmp_path / "trace.json"))
    assert len(trace["traceEvents"]) == len(events)
    # the committed answer of the reference's own analyze_bundle for exactly these bundles
    golden = json.load(open(os.path.join(HERE, "golden", "profile_diagnosis.json")))[case]
    assert golden["schema_version"] == 1
    cats = [d["category"] for d in golden["diagnostics"]]
    assert "bundle_schema_error" not in cats
    assert sorted(c for c in cats if c != "no_issues_detected") == sorted(_rules(events))
    launches = [e for e in events if e["event_type"] == "kernel_launch"]
    assert launches and all(e["kernel_symbol"] and e["metrics"]["device_ms"] > 0 for e in launches)


_GPU_CHILD = r"""
import json, os, sys
import numpy as np, torch
sys.path.insert(0, sys.argv[1])
from hdkx_aicompiler_b200 import plan, profiling, relay as R
rng = np.random.default_rng(3)
def const(*shape):
    return R.Constant(torch.from_numpy(rng.normal(0, 0.1, shape).astype(np.float32)).cuda())
x = R.Var("x", (4, 64, 28, 28), "float32")
c1 = R.Call("nn_relu", [R.Call("nn_conv2d", [x, const(64, 64, 3, 3), const(64)], R.Conv2DAttrs((1, 1), (1, 1), (1, 1), 1))])
g = R.Call("nn_flatten", [R.Call("nn_global_avg_pool2d", [c1])])
f = R.Function([x], R.Call("nn_gemm", [g, const(10, 64), const(10)], R.GemmAttrs(1.0, 1.0, 0, 1)))
xin = torch.from_numpy(rng.normal(0, 1, (4, 64, 28, 28)).astype(np.float32))
graph = plan.CompiledGraph(f, precision="bf16")
plain = graph.run(xin.cuda()).cpu()
graph.set_nvtx(True)
ranged = graph.run(xin.cuda()).cpu()
assert torch.equal(plain, ranged)
bundle = profiling.ProfileBundle(sys.argv[2], worker_id=0)
pr = profiling.ProfiledRun(graph, bundle)
dev = torch.empty_like(xin, device="cuda")
host_out = torch.empty(graph.out_shape, dtype=torch.float32).pin_memory()
pr.copy_to_device(xin.pin_memory(), dev)
out, run_id = pr.run(dev)
pr.copy_to_host(out, host_out)
assert torch.equal(host_out, plain)
bundle.write()
print(json.dumps({"launches": graph.num_launches, "labels": [l for l, _, _ in graph.launch_info()]}))
"""


@pytest.mark.gpu
def test_nvtx_ranges_and_profiled_run(tmp_path):
    probe = tmp_path / "nvtx_probe.so"
    subprocess.check_call(["gcc", "-shared", "-fPIC", "-O1", "-I/usr/local/cuda/include", os.path.join(HERE, "nvtx_probe.c"),
                           "-o", str(probe)])
    log = tmp_path / "nvtx.log"
    bundle_dir = tmp_path / "bundle"
    env = dict(os.environ, NVTX_INJECTION64_PATH=str(probe), KXC_NVTX_PROBE_LOG=str(log))
    res = subprocess.run([sys.executable, "-c", _GPU_CHILD, ROOT, str(bundle_dir)], env=env, capture_output=True, text=True,
                         timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    info = json.loads(res.stdout.strip().splitlines()[-1])
    lines = [l.rstrip("\n") for l in open(log)]
    # the run with ranges on: one outer range, one range per launch, properly nested
    pushes = [l[5:] for l in lines if l.startswith("push ")]
    assert pushes[0] == "kxc_b200_plan_run"
    assert pushes[1:1 + info["launches"]] == info["labels"]
    depth = 0
    for l in lines:
        depth += 1 if l.startswith("push ") else -1
        assert 0 <= depth <= 2
    assert depth == 0
    events = [json.loads(line) for line in open(bundle_dir / "events.jsonl")]
    kinds = [(e["component"], e["event_type"]) for e in events]
    assert kinds.count(("device_api", "copy")) == 2
    assert kinds.count(("runtime", "compiled_module_run")) == 1
    assert kinds.count(("kernel", "kernel_launch")) == info["launches"]
    assert [e["kernel_symbol"] for e in events if e["event_type"] == "kernel_launch"] == info["labels"]
    for ev in events:
        assert tuple(ev) == profiling.EVENT_KEYS
    run = next(e for e in events if e["event_type"] == "compiled_module_run")
    assert run["duration_ns"] > 0 and run["device"].startswith("cuda:")

"""The reference-side binding (adapter/): a translation unit compiled against the UNMODIFIED reference's headers and
linked with its objects and with libkxc_b200.so. The tests drive the reference's own entry points with the library's
kernels behind them:

  * CompiledKernel::operator() on a whole imported graph (src/codegen/compiled_kernel.cc:41-55): the `int32_t f(void**)`
    thunk, the packed argument order, device memory from the reference's CUDADeviceAPI, the exception on a non-zero return;
  * the reference's ExecutionPlan walked node by node, every KernelExecNode dispatched through its bound kernel_symbol
    (src/base/disco/executor.cc:122-157 is the placeholder this replaces);
  * a CCLBackend over NCCL against the reference's CpuCCLBackend (src/base/disco/ccl_cpu.cc:176-317).

The binary is built where a checkout of the reference is present (adapter/Makefile) and travels with the repository's
other built files; without it the tests skip."""
import os
import subprocess

import numpy as np
import pytest

from conftest import assert_bit_exact, assert_close

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEMO = os.path.join(ROOT, "adapter", "build", "adapter_demo")
GOLDEN = os.path.join(ROOT, "tests", "golden")
needs_demo = pytest.mark.skipif(not os.path.exists(DEMO), reason="adapter/build/adapter_demo is not built (needs the reference sources)")


def run_demo(*args, timeout=300):
    r = subprocess.run([DEMO, *args], capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, f"adapter_demo {' '.join(args)} failed:\n{r.stdout}\n{r.stderr}"
    return r.stdout


@needs_demo
def test_op_registry_carries_the_launch_attribute():
    """Every operator of the path has an FB200Launch attribute beside the reference's own FInferType / FRelayToTE, and its
    kernel_symbol resolves in the loaded library (no GPU needed)."""
    out = run_demo("registry")
    assert "registry ok" in out
    for op, sym in (("nn_conv2d", "kxc_b200_nn_conv2d"), ("nn_gemm", "kxc_b200_nn_gemm"), ("nn_max_pool2d", "kxc_b200_nn_max_pool2d")):
        assert f"{op} -> {sym} (resolved)" in out


def _golden_io(tmp_path):
    io = np.load(os.path.join(GOLDEN, "import_block_io.npz"))
    inp = tmp_path / "input.bin"
    io["input"].astype(np.float32).tofile(inp)
    return io, str(inp)


@needs_demo
@pytest.mark.gpu
@pytest.mark.parametrize("precision", ["fp32", "tf32"])
def test_compiled_kernel_runs_the_imported_graph(tmp_path, precision):
    io, inp = _golden_io(tmp_path)
    outp = str(tmp_path / "out.bin")
    out = run_demo("graph", os.path.join(GOLDEN, "import_block.json"), os.path.join(GOLDEN, "import_block.bin"), inp, outp, precision)
    assert "graph ok" in out and "error path: Kernel kxc_kernel_main returned error code" in out
    got = np.fromfile(outp, dtype=np.float32).reshape(io["output"].shape)
    if precision == "fp32":
        assert_bit_exact(got, io["output"], "CompiledKernel (fp32 plan) vs the reference's own output")
    else:
        assert_close(got, io["output"], 1e-2, "CompiledKernel (tf32 plan)")


@needs_demo
@pytest.mark.gpu
def test_execution_plan_nodes_dispatch_through_kernel_symbol(tmp_path):
    io, inp = _golden_io(tmp_path)
    outp = str(tmp_path / "out.bin")
    out = run_demo("plan", os.path.join(GOLDEN, "import_block.json"), os.path.join(GOLDEN, "import_block.bin"), inp, outp, "fp32")
    assert "plan ok" in out
    assert "nn_conv2d -> kxc_b200_nn_conv2d" in out and "add -> kxc_b200_add" in out
    got = np.fromfile(outp, dtype=np.float32).reshape(io["output"].shape)
    assert_bit_exact(got, io["output"], "ExecutionPlan executed node by node vs the reference's own output")


@needs_demo
@pytest.mark.gpu
def test_nccl_ccl_backend_matches_the_cpu_backend():
    import torch
    out = run_demo("ccl", "1")
    assert "ccl ok workers=1" in out
    if torch.cuda.device_count() >= 2:
        out = run_demo("ccl", "2")
        assert "ccl ok workers=2" in out and "gather_to_worker0 ok" in out

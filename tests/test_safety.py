"""The library's safety plumbing: the bounded device-side wait that every tensor-core kernel uses, the status
word it reports into, the once-per-device kernel set-up, and the threading contract of the per-operator entry
points (the reference calls the same kernel entry from several host threads: src/runtime/kernel_runner.cc:17-30)."""
import ctypes
import threading

import numpy as np
import pytest
import torch

from conftest import assert_bit_exact


def test_per_device_once_bookkeeping():
    """Host-only: the shared-memory opt-in is repeated once per device ordinal, retried after a failure."""
    from hdkx_aicompiler_b200 import _lib
    lib = _lib.load()
    assert lib.kxc_b200_selftest_per_device_once() == 0, _lib.last_error()


@pytest.mark.gpu
def test_bounded_wait_runs_out_and_is_reported():
    """A wait on a barrier nobody arrives on gives up after its limit (1 ms here): the kernel returns, the status
    word reads KXC_B200_ERR_DEVICE_WAIT, kxc_b200_device_status reports and clears it, and the context stays usable."""
    from hdkx_aicompiler_b200 import _lib, ops
    lib = _lib.load()
    assert ops.device_status() == 0
    stream = torch.cuda.current_stream().cuda_stream
    gave_up = ctypes.c_int32(-1)
    rc = lib.kxc_b200_selftest_bounded_wait(1_000_000, stream, ctypes.byref(gave_up))
    assert rc == 0, _lib.last_error()
    assert gave_up.value == 1
    st = ctypes.c_int32(0)
    rc = lib.kxc_b200_device_status(stream, ctypes.byref(st))
    assert rc == 5 and st.value == 5  # KXC_B200_ERR_DEVICE_WAIT
    assert "bounded wait" in _lib.last_error()
    with pytest.raises(_lib.KxcError):  # the Python mirror raises like the reference's CompiledKernel does
        lib.kxc_b200_selftest_bounded_wait(1_000_000, stream, ctypes.byref(gave_up))
        ops.device_status()
    assert ops.device_status() == 0  # cleared by the read
    # limits outside (0, 100 ms] are refused before anything is launched
    assert lib.kxc_b200_selftest_bounded_wait(0, stream, None) == 1
    assert lib.kxc_b200_selftest_bounded_wait(10**10, stream, None) == 1
    # the context is intact: a real tensor-core kernel still runs and leaves the word clean
    x = torch.ones(1, 64, 8, 8, device="cuda")
    w = torch.ones(64, 64, 1, 1, device="cuda")
    y = ops.nn_conv2d(x, w, precision="bf16")
    assert ops.device_status() == 0
    assert float(y.min()) == 64.0 and float(y.max()) == 64.0


@pytest.mark.gpu
def test_two_host_threads_share_the_entry_points():
    """Two host threads call per-operator entry points at the same time, each on its own stream: results equal the
    single-threaded ones bit for bit."""
    from hdkx_aicompiler_b200 import ops
    rng = np.random.default_rng(3)
    x = torch.from_numpy(rng.uniform(-1, 1, (4, 64, 28, 28)).astype(np.float32)).cuda()
    w = torch.from_numpy(rng.normal(0, 0.05, (128, 64, 3, 3)).astype(np.float32)).cuda()
    b = torch.from_numpy(rng.normal(0, 0.05, (128,)).astype(np.float32)).cuda()
    want_conv = ops.nn_conv2d(x, w, b, (1, 1), (1, 1), relu=True, precision="bf16").cpu().numpy()
    want_pool = ops.nn_max_pool2d(x, (3, 3), (2, 2), (1, 1, 1, 1)).cpu().numpy()
    want_relu = ops.nn_relu(x).cpu().numpy()
    torch.cuda.synchronize()
    errors, results = [], {}

    def worker(tid):
        try:
            torch.cuda.set_device(0)
            stream = torch.cuda.Stream()
            out = []
            with torch.cuda.stream(stream):
                for _ in range(20):
                    c = ops.nn_conv2d(x, w, b, (1, 1), (1, 1), relu=True, precision="bf16")
                    p = ops.nn_max_pool2d(x, (3, 3), (2, 2), (1, 1, 1, 1))
                    r = ops.nn_relu(x)
                    out = [c, p, r]
                stream.synchronize()
            results[tid] = [t.cpu().numpy() for t in out]
        except Exception as e:  # noqa: BLE001
            errors.append((tid, repr(e)))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert ops.device_status() == 0
    for tid in range(2):
        assert_bit_exact(results[tid][0], want_conv, f"thread {tid} conv")
        assert_bit_exact(results[tid][1], want_pool, f"thread {tid} pool")
        assert_bit_exact(results[tid][2], want_relu, f"thread {tid} relu")


@pytest.mark.gpu
def test_two_host_threads_on_one_plan_are_serialised():
    """One plan = one run in flight: calls from two threads on the same stream are serialised by the plan's mutex
    and every result equals the single-threaded one."""
    from hdkx_aicompiler_b200 import plan, relay as R
    rng = np.random.default_rng(4)
    wt = torch.from_numpy(rng.normal(0, 0.05, (64, 16, 3, 3)).astype(np.float32)).cuda()
    bs = torch.from_numpy(rng.normal(0, 0.05, (64,)).astype(np.float32)).cuda()
    xv = R.Var("input", (2, 16, 12, 12))
    func = R.Function([xv], R.Call("nn_relu", [R.Call("nn_conv2d", [xv, R.Constant(wt), R.Constant(bs)],
                                                      R.Conv2DAttrs((1, 1), (1, 1, 1, 1), (1, 1), 1))]))
    g = plan.CompiledGraph(func, "bf16")
    xs = [torch.from_numpy(rng.uniform(-1, 1, (2, 16, 12, 12)).astype(np.float32)).cuda() for _ in range(2)]
    want = [g.run(x).cpu().numpy() for x in xs]
    stream = torch.cuda.Stream()
    errors, got = [], {}

    def worker(tid):
        try:
            torch.cuda.set_device(0)
            with torch.cuda.stream(stream):
                for _ in range(10):
                    out = g.run(xs[tid])
                stream.synchronize()
            got[tid] = out.cpu().numpy()
        except Exception as e:  # noqa: BLE001
            errors.append((tid, repr(e)))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for tid in range(2):
        assert_bit_exact(got[tid], want[tid], f"thread {tid}")

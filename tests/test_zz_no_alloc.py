"""kxc_b200_nn_conv2d_static_scratch: the convolution entry point for hosts that may not allocate.

Collected last on purpose (file name): a run that stops at the first failure has then already run
every other test. The test is self-contained, so it also passes alone in a fresh process.

It calls the entry point through the C ABI twice in a row with different operands (the second call
reuses the library's fixed workspace with the first call's bytes still in it) and checks each result
against the regular, allocating entry point, which runs the same kernels on the same values, and against
the CPU oracle on identically rounded operands. A further pair of calls checks the claim itself: the
device's free memory is the same before and after a warmed-up call, and the status word stays clean.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, fn, x, w, b, res, out, desc_args, stream):
    from hdkx_aicompiler_b200 import _lib
    desc = _lib.Conv2dDesc(*desc_args)
    args = _lib.packed(x.data_ptr(), w.data_ptr(), b.data_ptr(), res.data_ptr(), out.data_ptr())
    rc = fn(args, desc, stream)
    return rc


@pytest.mark.parametrize("precision", ["bf16", "tf32"])
def test_static_scratch_conv_matches_allocating_entry_point(precision):
    from hdkx_aicompiler_b200 import _lib
    assert torch.cuda.is_available()
    lib = _lib.load()
    prec = {"bf16": _lib.PREC_BF16, "tf32": _lib.PREC_TF32}[precision]
    flags = _lib.BIAS | _lib.RESIDUAL | _lib.RELU
    stream = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator(device="cuda").manual_seed(5)
    # two different problems back to back: the second is smaller, so stale bytes of the first remain behind it
    for (N, C, H, W, O, K, s, p) in [(4, 64, 28, 28, 128, 3, 1, 1), (2, 24, 15, 13, 40, 3, 2, 1)]:
        OH, OW = (H + 2 * p - K) // s + 1, (W + 2 * p - K) // s + 1
        x = torch.empty(N, C, H, W, device="cuda").uniform_(-1, 1, generator=gen)
        w = torch.empty(O, C, K, K, device="cuda").normal_(0, (2.0 / (C * K * K)) ** 0.5, generator=gen)
        b = torch.empty(O, device="cuda").normal_(0, 0.05, generator=gen)
        res = torch.empty(N, O, OH, OW, device="cuda").uniform_(-1, 1, generator=gen)
        out_static = torch.full((N, O, OH, OW), float("nan"), device="cuda")
        out_ref = torch.full((N, O, OH, OW), float("nan"), device="cuda")
        d = (N, C, H, W, O, K, K, s, s, p, p, 1, 1, flags, prec)
        rc = _call(lib, lib.kxc_b200_nn_conv2d_static_scratch, x, w, b, res, out_static, d, stream)
        assert rc == 0, _lib.last_error()
        rc = _call(lib, lib.kxc_b200_nn_conv2d, x, w, b, res, out_ref, d, stream)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        a, r = out_static.cpu().numpy(), out_ref.cpu().numpy()
        assert np.isfinite(a).all()
        # same kernels, same operand values, same summation order: the tolerance of the tensor-core tests
        # (2e-5 on the reference's |a-r|/max(1,|r|) metric) is in fact met with equality
        err = np.abs(a - r) / np.maximum(1.0, np.abs(r))
        assert err.max() <= 2e-5, err.max()
        assert np.array_equal(a, r)
        # and against the CPU oracle on the same rounded operands (only the fp32 summation order differs)
        from oracle import port
        rnd = port.round_bf16 if precision == "bf16" else port.round_tf32
        exp = port.relu(port.add(port.conv2d(rnd(x.cpu().numpy()), rnd(w.cpu().numpy()), b.cpu().numpy(), (s, s), (p, p)),
                                 res.cpu().numpy()))
        err = np.abs(a - exp) / np.maximum(1.0, np.abs(exp))
        assert err.max() <= 2e-5, err.max()
    # a wait that ran out in these kernels would show here: their status word is read together with the regular one
    from hdkx_aicompiler_b200 import ops
    assert ops.device_status() == 0


def test_static_scratch_call_allocates_nothing():
    """Free device memory is the same before and after a warmed-up call (and its kernels have finished)."""
    from hdkx_aicompiler_b200 import _lib, ops
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    N, C, H, W, O, K = 2, 32, 20, 20, 64, 3
    x = torch.rand(N, C, H, W, device="cuda")
    w = torch.rand(O, C, K, K, device="cuda")
    b = torch.rand(O, device="cuda")
    res = torch.rand(N, O, H, W, device="cuda")
    out = torch.empty(N, O, H, W, device="cuda")
    d = (N, C, H, W, O, K, K, 1, 1, 1, 1, 1, 1, _lib.BIAS | _lib.RESIDUAL | _lib.RELU, _lib.PREC_BF16)
    assert _call(lib, lib.kxc_b200_nn_conv2d_static_scratch, x, w, b, res, out, d, stream) == 0, _lib.last_error()  # warm-up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert _call(lib, lib.kxc_b200_nn_conv2d_static_scratch, x, w, b, res, out, d, stream) == 0, _lib.last_error()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, (free_before, free_after)
    assert ops.device_status() == 0


def test_static_scratch_rejects_oversize():
    from hdkx_aicompiler_b200 import _lib
    lib = _lib.load()
    cap = lib.kxc_b200_static_scratch_bytes()
    assert cap == 32 * 1024 * 1024
    N, C, H, W, O = 64, 64, 56, 56, 64  # 64*56*56*64*2 B = 25.7 MB activations per 64 images -> 2 x that at N=128
    N = 128
    x = torch.zeros(1, device="cuda")  # never dereferenced: the size check comes first
    desc = _lib.Conv2dDesc(N, C, H, W, O, 3, 3, 1, 1, 1, 1, 1, 1, 0, _lib.PREC_BF16)
    args = _lib.packed(x.data_ptr(), x.data_ptr(), x.data_ptr())
    rc = lib.kxc_b200_nn_conv2d_static_scratch(args, desc, None)
    assert rc == 6  # KXC_B200_ERR_NOMEM
    assert "static scratch holds" in _lib.last_error()

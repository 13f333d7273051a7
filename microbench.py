"""Per-kernel measurements for the benchmark configurations that are not the headline number:

  config 1  fused conv2d + bias + ReLU, 1x64x56x56 (*) 64x64x3x3          (tensor / launch bound)
  config 2  max_pool2d 3x3 s2 p1 on 32x64x112x112 -> add -> relu            (HBM bound)
  config 5  int8 convolution sweep over the 11 distinct ResNet-18 shapes at N=256, requantize + ReLU
  config t  transpose / cast / softmax / reduce_mean / matmul on the operator ABI (the formats either side of the path)

    python microbench.py [--config 1|2|3|5|t|all] [--iters 20]

  config 3  ResNet-18 fp32/tf32 at batch 32 through the plan executor (tf32, tf32x3 and the bit-exact fp32 mode)

bench.py calls config1_plan / config2 / config3 of this file after the headline timing and puts their figures into its
JSON line (`hbm_kernels`, `config1`, `config3`). Prints one JSON line per measured kernel: CUDA-event time (L2 flushed between iterations by writing a
256 MB buffer), achieved GB/s or TOP/s and the fraction of the measured peak in MEASURED_PEAKS.json
(copy bandwidth / bf16 GEMM; int8 is reported against 2x the bf16 figure, the nominal ratio).
Inputs are synthetic with the configurations' shapes and value distributions.
"""
import argparse
import json
import os

import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from hdkx_aicompiler_b200 import ops, resnet18  # noqa: E402


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return p["hbm_gbs"], p["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def timeit(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return float(np.median(ts))


def timeit_rotating(fns, iters, flush):
    """Per-launch time of len(fns) launches issued back to back between ONE event pair, each on its own input buffers
    (together far larger than L2, so no launch finds its input cached). A single 15-30 us launch timed alone carries the
    event pair and an idle-GPU launch (about 5 us); this form amortizes them."""
    for f in fns:
        f()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for f in fns:
            f()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) / len(fns))
    return float(np.median(ts))


QUIET = False


def emit(**kw):
    """One JSON line per measurement (unless a caller collects the returned dicts itself)."""
    if not QUIET:
        print(json.dumps(kw), flush=True)
    return kw


def config1(iters, flush, hbm, tf, src):
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.empty(1, 64, 56, 56, device="cuda").uniform_(-1, 1, generator=g)
    w = torch.empty(64, 64, 3, 3, device="cuda").normal_(0, (2 / 576) ** 0.5, generator=g)
    b = torch.empty(64, device="cuda").normal_(0, 0.01, generator=g)
    out = torch.empty(1, 64, 56, 56, device="cuda")
    flops = 2 * 64 * 56 * 56 * 64 * 9
    for prec in ("fp32", "tf32", "bf16"):
        ms = timeit(lambda: ops.nn_conv2d(x, w, b, (1, 1), (1, 1), relu=True, precision=prec, out=out), iters, flush)
        emit(config=1, kernel=f"nn_conv2d+bias+relu {prec} (NCHW fp32 in/out, includes operand conversion)", ms=ms,
             tflops=flops / ms / 1e9, frac_of_bf16_peak=flops / ms / 1e9 / tf, peak_source=src)


    return config1_plan(iters, flush, hbm, tf, src)


def config1_plan(iters, flush, hbm, tf, src):
    """Config 1 inside a plan: operands resident in the kernels' layout, one CUDA-graph replay per call (input conversion,
    the row-stacked tensor-core kernel with fused bias + ReLU, conversion of the result back)."""
    from hdkx_aicompiler_b200 import plan, relay as R
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.empty(1, 64, 56, 56, device="cuda").uniform_(-1, 1, generator=g)
    w = torch.empty(64, 64, 3, 3, device="cuda").normal_(0, (2 / 576) ** 0.5, generator=g)
    b = torch.empty(64, device="cuda").normal_(0, 0.01, generator=g)
    out = torch.empty(1, 64, 56, 56, device="cuda")
    flops = 2 * 64 * 56 * 56 * 64 * 9
    xv = R.Var("input", (1, 64, 56, 56))
    func = R.Function([xv], R.Call("nn_relu", [R.Call("nn_conv2d", [xv, R.Constant(w), R.Constant(b)],
                                                        R.Conv2DAttrs((1, 1), (1, 1, 1, 1), (1, 1), 1))]))
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        g = plan.CompiledGraph(func, "bf16", cuda_graph=True)
        ms = timeit(lambda: g.run(x, out=out), iters, flush)
        _, per = g.run_timed(x, out=out)
    names = [i[0].split()[0] for i in g.launch_info()]
    return emit(config=1, kernel="plan bf16, CUDA-graph replay: " + " + ".join(names), ms=ms, tflops=flops / ms / 1e9,
                frac_of_bf16_peak=flops / ms / 1e9 / tf, launch_ms=dict(zip(names, [round(v, 4) for v in per])), peak_source=src)


def config2(iters, flush, hbm, tf, src):
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.empty(32, 64, 112, 112, device="cuda").uniform_(-1, 1, generator=g)
    res = torch.empty(32, 64, 56, 56, device="cuda").uniform_(-1, 1, generator=g)
    out = torch.empty_like(res)
    cases = [
        ("max_pool2d_add_relu (fused chain)", 154.14e6, lambda: ops.max_pool2d_add_relu(x, res, (3, 3), (2, 2), (1, 1, 1, 1), out=out)),
        ("nn_max_pool2d", 128.45e6, lambda: ops.nn_max_pool2d(x, (3, 3), (2, 2), (1, 1, 1, 1))),
        ("add", 77.07e6, lambda: ops.add(res, out)),
        ("nn_relu", 51.38e6, lambda: ops.nn_relu(res)),
    ]
    # the same byte counts moved by the driver's device-to-device copy, as the bar a kernel of this size can reach
    for nbytes in (154.14e6, 128.45e6, 77.07e6, 51.38e6):
        n = int(nbytes // 8)
        src_t = torch.empty(n, dtype=torch.float32, device="cuda").normal_()
        dst_t = torch.empty_like(src_t)
        cases.append((f"reference: copy_ of {nbytes / 2e6:.1f} MB (same bytes read + written)", nbytes, lambda d=dst_t, s_=src_t: d.copy_(s_)))
    results = []
    for name, nbytes, fn in cases:
        ms = timeit(fn, iters, flush)
        results.append(emit(config=2, kernel=name, form="one launch between two events", ms=ms, algorithmic_bytes=nbytes,
                            gbs=nbytes / ms / 1e6, frac_of_hbm_peak=nbytes / ms / 1e6 / hbm, peak_source=src))
    # the same four kernels, eight launches back to back on eight different input sets (8 x 51-154 MB, L2 is 126 MB)
    sets = 8
    xs = [torch.empty_like(x).uniform_(-1, 1, generator=g) for _ in range(sets)]
    rs = [torch.empty_like(res).uniform_(-1, 1, generator=g) for _ in range(sets)]
    os_ = [torch.empty_like(res) for _ in range(sets)]
    # straight through the C ABI with descriptors and argument lists built once: the Python wrappers in ops.py cost
    # 10-25 us per call, more than these kernels run
    from hdkx_aicompiler_b200 import _lib
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    pool_desc = _lib.Pool2dDesc(32, 64, 112, 112, 3, 3, 2, 2, 1, 1, 1, 1, 0)
    add_desc = _lib.AddDesc()
    add_desc.rank_a = add_desc.rank_b = 4
    for i, d in enumerate(res.shape):
        add_desc.shape_a[i] = add_desc.shape_b[i] = d
    ptr = lambda t: t.data_ptr()  # noqa: E731
    chain_args = [_lib.packed(ptr(xs[i]), ptr(rs[i]), ptr(os_[i])) for i in range(sets)]
    pool_args = [_lib.packed(ptr(xs[i]), ptr(os_[i])) for i in range(sets)]
    add_args = [_lib.packed(ptr(rs[i]), ptr(rs[(i + 1) % sets]), ptr(os_[i])) for i in range(sets)]
    relu_args = [_lib.packed(ptr(rs[i]), ptr(os_[i])) for i in range(sets)]
    nres = res.numel()
    rotating = [
        ("max_pool2d_add_relu (fused chain)", 154.14e6, [lambda a=a: lib.kxc_b200_max_pool2d_add_relu(a, pool_desc, stream) for a in chain_args]),
        ("nn_max_pool2d", 128.45e6, [lambda a=a: lib.kxc_b200_nn_max_pool2d(a, pool_desc, stream) for a in pool_args]),
        ("add", 77.07e6, [lambda a=a: lib.kxc_b200_add(a, add_desc, stream) for a in add_args]),
        ("nn_relu", 51.38e6, [lambda a=a: lib.kxc_b200_nn_relu(a, nres, stream) for a in relu_args]),
        ("reference: copy_ of 64.2 MB", 128.45e6, [lambda i=i: xs[i].view(-1)[:16056320].copy_(xs[(i + 1) % sets].view(-1)[:16056320]) for i in range(sets)]),
    ]
    for name, nbytes, fns in rotating:
        ms = timeit_rotating(fns, iters, flush)
        results.append(emit(config=2, kernel=name, form=f"{sets} launches back to back on rotating buffers, per launch", ms=ms,
                            algorithmic_bytes=nbytes, gbs=nbytes / ms / 1e6, frac_of_hbm_peak=nbytes / ms / 1e6 / hbm, peak_source=src))
    return results


def config3(iters, flush, hbm, tf, src):
    """ResNet-18 at batch 32 (the fp32/tf32 configuration): device-timed CUDA-graph replays per precision."""
    from hdkx_aicompiler_b200 import plan
    N = 32
    weights = resnet18.make_weights(seed=0)
    x = torch.empty(N, 3, 224, 224, device="cuda").normal_(0, 1, generator=torch.Generator(device="cuda").manual_seed(3))
    results = []
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for prec, reps in (("tf32", max(3, iters)), ("tf32x3", max(3, iters)), ("fp32", 2)):
            g = plan.CompiledGraph(resnet18.build(N, weights, to_constant=lambda a: torch.from_numpy(a).cuda()), prec, cuda_graph=True)
            out = torch.empty(g.out_shape, device="cuda")
            ms = timeit(lambda: g.run(x, out=out), reps, flush)
            ops.device_status()
            results.append(emit(config=3, kernel=f"resnet18 batch {N} plan {prec}, CUDA-graph replay", ms=ms, img_per_s=N / ms * 1e3,
                                launches=g.num_launches, tflops=3.628147e9 * N / ms / 1e9))
            del g
    return results


def config5(iters, flush, hbm, tf, src):
    rng = np.random.default_rng(0)
    N = 256
    for name, cin, cout, k, s, p, h, _ in resnet18.CONV_SHAPES:
        x = torch.from_numpy(np.clip(np.round(rng.normal(0, 32, (N, cin, h, h))), -128, 127).astype(np.int8)).cuda()
        wf = rng.normal(0, np.sqrt(2.0 / (cin * k * k)), (cout, cin, k, k))
        scale = np.abs(wf).reshape(cout, -1).max(axis=1) / 127.0
        w = torch.from_numpy(np.clip(np.round(wf / scale[:, None, None, None]), -127, 127).astype(np.int8)).cuda()
        b = torch.from_numpy(rng.integers(-1024, 1025, (cout,)).astype(np.int32)).cuda()
        m = torch.from_numpy(rng.integers(2 ** 30, 2 ** 31, (cout,)).astype(np.int64).astype(np.int32)).cuda()
        sh = torch.from_numpy(rng.integers(8, 16, (cout,)).astype(np.int32)).cuda()
        oh = (h + 2 * p - k) // s + 1
        ops_count = 2 * N * cout * oh * oh * cin * k * k
        ms = timeit(lambda: ops.nn_conv2d_s8(x, w, b, m, sh, (s, s), (p, p), relu=True), max(3, iters // 4), flush)
        same = bool(torch.equal(ops.nn_conv2d_s8(x, w, b, m, sh, (s, s), (p, p), relu=True),
                                ops.nn_conv2d_s8(x, w, b, m, sh, (s, s), (p, p), relu=True, simt=True)))
        emit(config=5, kernel=f"nn_conv2d_s8 {name} N={N} (NCHW int8 in/out, includes operand conversion)", ms=ms,
             tops=ops_count / ms / 1e9, frac_of_2x_bf16_peak=ops_count / ms / 1e9 / (2 * tf), tcgen05_equals_cuda_core_kernel=same,
             peak_source=src)
        # the same convolution with the tensors resident in the kernel's layout (NHWC int8, channels padded to the
        # K-block granularity), as between the layers of a quantized network: the kernel alone
        # (a first layer of <= 8 channels keeps its raw NHWC pixels: the library packs them for its direct stem kernel)
        cp = cin if cin <= 8 else 32 if cin <= 32 else (64 if cin <= 64 else (cin + 127) // 128 * 128)
        xh = torch.zeros((N, h, h, cp), dtype=torch.int8, device="cuda")
        xh[..., :cin] = x.permute(0, 2, 3, 1)
        wh = torch.zeros((cout, k, k, cp), dtype=torch.int8, device="cuda")
        wh[..., :cin] = w.permute(0, 2, 3, 1)
        ms2 = timeit(lambda: ops.nn_conv2d_s8(xh, wh, b, m, sh, (s, s), (p, p), relu=True, nhwc=True), max(3, iters // 4), flush)
        same2 = bool(torch.equal(ops.nn_conv2d_s8(xh, wh, b, m, sh, (s, s), (p, p), relu=True, nhwc=True).permute(0, 3, 1, 2),
                                 ops.nn_conv2d_s8(x, w, b, m, sh, (s, s), (p, p), relu=True)))
        emit(config=5, kernel=f"nn_conv2d_s8 {name} N={N} (NHWC int8 resident, kernel only)", ms=ms2, tops=ops_count / ms2 / 1e9,
             frac_of_2x_bf16_peak=ops_count / ms2 / 1e9 / (2 * tf), equals_reference_layout_call=same2, peak_source=src)
    ops.device_status()


def config_transform(iters, flush, hbm, tf, src):
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.empty(32, 64, 112, 112, device="cuda").uniform_(-1, 1, generator=g)
    nb = x.numel() * 4.0
    xs8 = ops.cast(x * 100, "int8")
    logits = torch.empty(65536, 1000, device="cuda").normal_(generator=g)
    feat = torch.empty(1024, 512, 7, 7, device="cuda").normal_(generator=g)
    cases = [
        ("transpose NCHW -> NHWC (0,2,3,1)", 2 * nb, lambda: ops.transpose(x, (0, 2, 3, 1))),
        ("transpose NHWC -> NCHW (0,3,1,2)", 2 * nb, lambda: ops.transpose(x.view(32, 112, 112, 64), (0, 3, 1, 2))),
        ("transpose batch <-> channel (1,0,2,3)", 2 * nb, lambda: ops.transpose(x, (1, 0, 2, 3))),
        ("transpose reverse (3,2,1,0)", 2 * nb, lambda: ops.transpose(x, (3, 2, 1, 0))),
        ("cast float32 -> int32", 2 * nb, lambda: ops.cast(x, "int32")),
        ("cast float32 -> int8", 1.25 * nb, lambda: ops.cast(x, "int8")),
        ("cast int8 -> float32", 1.25 * nb, lambda: ops.cast(xs8, "float32")),
        ("cast float32 -> float64", 3 * nb, lambda: ops.cast(x, "float64")),
        ("softmax 65536 x 1000 (last axis)", 2.0 * logits.numel() * 4, lambda: ops.softmax(logits, -1)),
        ("reduce_mean 1024x512x7x7 over (2,3)", feat.numel() * 4.0 + 1024 * 512 * 4, lambda: ops.reduce_mean(feat, (2, 3), True)),
    ]
    dst = torch.empty_like(x)
    cases.append((f"reference: copy_ of {nb / 1e6:.1f} MB (same bytes as a transpose)", 2 * nb, lambda: dst.copy_(x)))
    for name, nbytes, fn in cases:
        ms = timeit(fn, iters, flush)
        emit(config="t", kernel=name, ms=ms, algorithmic_bytes=nbytes, gbs=nbytes / ms / 1e6, frac_of_hbm_peak=nbytes / ms / 1e6 / hbm,
             peak_source=src)
    a = torch.empty(4096, 4096, device="cuda").normal_(generator=g)
    b = torch.empty(4096, 4096, device="cuda").normal_(generator=g)
    def four(prec):  # four calls per sample: a single call after an idle GPU mostly measures the host's launch path
        for _ in range(4):
            ops.matmul(a, b, precision=prec)

    for prec in ("bf16", "tf32"):
        ms = timeit(lambda: four(prec), iters, flush) / 4
        fl = 2.0 * 4096 ** 3
        emit(config="t", kernel=f"matmul 4096x4096x4096 {prec} (fp32 operands converted inside the call)", ms=ms, flops=fl,
             tflops=fl / ms / 1e9, frac_of_tensor_peak=fl / ms / 1e9 / (tf if prec == "bf16" else tf / 2), peak_source=src)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="all", help="1, 2, 3, 5, t or all")
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    assert torch.cuda.is_available(), "needs a GPU"
    hbm, tf, src = peaks()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    for c, fn in (("1", config1), ("2", config2), ("3", config3), ("5", config5), ("t", config_transform)):
        if args.config in ("all", c):
            fn(args.iters, flush, hbm, tf, src)


if __name__ == "__main__":
    main()

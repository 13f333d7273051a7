"""CPU tests of the oracle: the port against the reference's golden vectors and, bit for bit, against
the C text the unmodified reference compiler emits (oracle/_ref/ref_emit, when built)."""
import numpy as np
import pytest

from conftest import assert_bit_exact
from oracle import port, ref

f32 = np.float32


def near(a, e, tol=1e-4):  # ExpectNear of test/op_numeric_llvm_test.cpp:26-37
    a, e = np.asarray(a, f32).ravel(), np.asarray(e, f32).ravel()
    assert a.shape == e.shape and np.all(np.abs(a - e) <= tol), (a, e)


# ---- golden vectors of the reference's own numeric tests (test/op_numeric_llvm_test.cpp) ----------
@pytest.mark.parametrize("impl", ["port", "ref"])
def test_reference_golden_vectors(impl):
    if impl == "ref" and not ref.available():
        pytest.skip("oracle/_ref/ref_emit not built")
    m = port if impl == "port" else ref
    A = lambda v, s: np.array(v, dtype=f32).reshape(s)  # noqa: E731
    # TestAdd :59-70 (broadcast [2,3] + [3])
    near(m.add(A([1, 2, 3, 4, 5, 6], (2, 3)), A([10, 20, 30], (3,))), [11, 22, 33, 14, 25, 36])
    # TestDense :135-147
    near(m.dense(A([1, 2, 3, 4, 5, 6], (2, 3)), A([1, 0, 1, 0, 1, 1], (2, 3))), [4, 5, 10, 11])
    # TestGemm :149-163 (alpha=beta=1, transB=1)
    near(m.gemm(A([1, 2, 3, 4, 5, 6], (2, 3)), A([1, 0, 0, 0, 1, 0, 0, 0, 1, 1, 1, 1], (4, 3)), A([10, 20, 30, 40], (4,)),
                1.0, 1.0, 0, 1), [11, 22, 33, 46, 14, 25, 36, 55])
    # TestRelu :165-174
    near(m.relu(A([-2, -0.5, 0, 1, 2, -3], (6,))), [0, 0, 0, 1, 2, 0])
    # TestConv2D :176-189 (1x1x3x3 * 1x1x2x2, stride 1, no padding)
    near(m.conv2d(A(range(1, 10), (1, 1, 3, 3)), A([1, 0, 0, 1], (1, 1, 2, 2))), [6, 8, 12, 14])
    # TestMaxPool2D :191-203 / TestAvgPool2D :205-217 (2x2 window, stride 2)
    x = A(range(1, 17), (1, 1, 4, 4))
    near(m.max_pool2d(x, (2, 2), (2, 2), (0, 0, 0, 0)), [6, 8, 14, 16])
    near(m.avg_pool2d(x, (2, 2), (2, 2), (0, 0, 0, 0)), [3.5, 5.5, 11.5, 13.5])
    # TestGlobalAvgPool2D :219-229
    near(m.global_avg_pool2d(A([1, 2, 3, 4, 10, 20, 30, 40], (1, 2, 2, 2))), [2.5, 25.0])
    # TestModelAddChain :313-325
    xx, yy = A([1, 2, 3, 4], (4,)), A([10, 20, 30, 40], (4,))
    near(m.add(m.add(xx, yy), yy), [21, 42, 63, 84])
    # TestModelMLP :327-345  dense -> relu -> dense
    h = m.relu(m.dense(A([1, 2], (1, 2)), A([1, 0, 0, 1, 1, 1], (3, 2))))
    near(m.dense(h, A([1, 1, 1, 1, 0, -1], (2, 3))), [6, -2])
    # TestModelCNN :347-371  conv -> relu -> gap -> flatten -> dense
    c = m.relu(m.conv2d(A(range(1, 10), (1, 1, 3, 3)), A([1, 0, 0, 1], (1, 1, 2, 2))))
    g = m.global_avg_pool2d(c).reshape(1, 1)
    near(m.dense(g, A([1, 2], (2, 1))), [10, 20])


def test_shape_rules():
    # test/infer_type_test.cpp:106-132: conv {1,3,32,32} * {8,3,3,3} s2 p1 -> {1,8,16,16}; pool 2x2 s2 -> {1,8,8,8}
    assert port.conv_out_dim(32, 3, 2, 1) == 16
    assert port.pool_out_dim(16, 2, 2, 0, 0) == 8
    assert port.pool_out_dim(112, 3, 2, 1, 1) == 56
    assert port.pool_out_dim(7, 2, 2, 0, 0, True) == 4 and port.pool_out_dim(7, 2, 2, 0, 0, False) == 3


needs_ref = pytest.mark.skipif(not ref.available(), reason="oracle/_ref/ref_emit not built")


@needs_ref
@pytest.mark.parametrize("stride,pad,dil", [((1, 1), (1, 1), (1, 1)), ((2, 2), (1, 1), (1, 1)), ((2, 1), (0, 2), (1, 2)),
                                            ((2, 2), (3, 3), (1, 1))])
def test_port_conv_matches_reference_bits(rng, stride, pad, dil):
    x = rng.uniform(-1, 1, (2, 5, 13, 11)).astype(f32)
    w = rng.normal(0, 0.2, (7, 5, 3, 3)).astype(f32)
    b = rng.normal(0, 0.1, (7,)).astype(f32)
    assert_bit_exact(port.conv2d(x, w, b, stride, pad, dil), ref.conv2d(x, w, b, stride, pad, dil), "conv+bias")
    assert_bit_exact(port.conv2d(x, w, None, stride, pad, dil), ref.conv2d(x, w, None, stride, pad, dil), "conv")
    assert_bit_exact(port.relu(port.conv2d(x, w, b, stride, pad, dil)), ref.conv2d(x, w, b, stride, pad, dil, relu=True),
                     "conv+bias+relu")


@needs_ref
def test_port_conv_int32_matches_reference(rng):
    x = rng.integers(-128, 128, (2, 6, 9, 9)).astype(np.int32)
    w = rng.integers(-128, 128, (5, 6, 3, 3)).astype(np.int32)
    b = rng.integers(-1024, 1024, (5,)).astype(np.int32)
    expected = ref.conv2d(x, w, b, (2, 2), (1, 1))
    assert np.array_equal(port.conv2d_i32(x, w, b, (2, 2), (1, 1)), expected)
    # the int8 path's accumulators are the reference's nn_conv2d on the widened values
    mult = rng.integers(2 ** 30, 2 ** 31, (5,)).astype(np.int64).astype(np.int32)
    shift = rng.integers(8, 16, (5,)).astype(np.int32)
    _, acc = port.conv2d_s8_requant(x.astype(np.int8), w.astype(np.int8), b, mult, shift, True, (2, 2), (1, 1),
                                    return_acc=True)
    assert np.array_equal(acc, expected)


@needs_ref
def test_port_elementwise_pool_dense_match_reference_bits(rng):
    x = rng.uniform(-1, 1, (2, 3, 12, 10)).astype(f32)
    x[0, 0, 0, 0] = -0.0
    x[0, 0, 0, 1] = np.nan
    x[0, 0, 0, 2] = np.inf
    x[0, 0, 0, 3] = -np.inf
    assert_bit_exact(port.relu(x), ref.relu(x), "relu")
    y = rng.uniform(-1, 1, x.shape).astype(f32)
    assert_bit_exact(port.add(x, y), ref.add(x, y), "add")
    assert_bit_exact(port.add(x, y[:, :, :1, :].copy()), ref.add(x, y[:, :, :1, :].copy()), "add broadcast")
    assert_bit_exact(port.add(x, y[0, 0, 0].copy()), ref.add(x, y[0, 0, 0].copy()), "add rank-1 broadcast")
    for k, s, p, ceil in [((3, 3), (2, 2), (1, 1, 1, 1), False), ((2, 2), (2, 2), (0, 0, 0, 0), False),
                          ((3, 2), (2, 1), (1, 0, 0, 1), True), ((3, 3), (1, 1), (1, 1, 1, 1), False)]:
        assert_bit_exact(port.max_pool2d(x, k, s, p, ceil), ref.max_pool2d(x, k, s, p, ceil), f"max_pool {k}{s}{p}")
        xf = np.nan_to_num(x, nan=0.5, posinf=2.0, neginf=-2.0)
        assert_bit_exact(port.avg_pool2d(xf, k, s, p, ceil), ref.avg_pool2d(xf, k, s, p, ceil), f"avg_pool {k}{s}{p}")
    assert_bit_exact(port.global_avg_pool2d(y), ref.global_avg_pool2d(y), "gap")
    a = rng.normal(size=(5, 37)).astype(f32)
    b = rng.normal(size=(11, 37)).astype(f32)
    c = rng.normal(size=(11,)).astype(f32)
    assert_bit_exact(port.dense(a, b), ref.dense(a, b), "dense")
    assert_bit_exact(port.gemm(a, b, c, 1.0, 1.0, 0, 1), ref.gemm(a, b, c, 1.0, 1.0, 0, 1), "gemm")
    assert_bit_exact(port.gemm(a, b, c, 0.5, 2.0, 0, 1), ref.gemm(a, b, c, 0.5, 2.0, 0, 1), "gemm alpha beta")
    bt = np.ascontiguousarray(b.T)
    assert_bit_exact(port.gemm(a, bt, c, 1.0, 1.0, 0, 0), ref.gemm(a, bt, c, 1.0, 1.0, 0, 0), "gemm transB=0")


@needs_ref
def test_port_chain_matches_reference_bits(rng):
    x = rng.uniform(-1, 1, (2, 4, 16, 16)).astype(f32)
    res = rng.uniform(-1, 1, (2, 4, 8, 8)).astype(f32)
    got = port.relu(port.add(port.max_pool2d(x, (3, 3), (2, 2), (1, 1, 1, 1)), res))
    assert_bit_exact(got, ref.pool_add_relu(x, res), "pool->add->relu")


def test_requantize_definition():
    # round half toward +inf, saturation, fused relu
    assert port.requant_one(3, 1 << 30, 8, False) == 0         # 3 * 2^30 / 2^39 = 0.0059
    assert port.requant_one(256, 1 << 30, 8, False) == 1       # 0.5 -> 1 (half up)
    assert port.requant_one(-256, 1 << 30, 8, False) == 0      # -0.5 -> 0 (toward +inf)
    assert port.requant_one(-257, 1 << 30, 8, False) == -1
    assert port.requant_one(10 ** 6, (1 << 31) - 1, 8, False) == 127
    assert port.requant_one(-10 ** 6, (1 << 31) - 1, 8, False) == -128
    assert port.requant_one(-10 ** 6, (1 << 31) - 1, 8, True) == 0
    rng = np.random.default_rng(1)
    for _ in range(2000):
        acc = int(rng.integers(-2 ** 31, 2 ** 31))
        m = int(rng.integers(2 ** 30, 2 ** 31))
        s = int(rng.integers(8, 16))
        relu = bool(rng.integers(0, 2))
        q = (acc * m + (1 << (30 + s))) >> (31 + s)          # Python ints: exact, floor shift
        q = min(max(q, 0 if relu else -128), 127)
        assert port.requant_one(acc, m, s, relu) == q


def test_rounding_helpers():
    import torch
    x = np.random.default_rng(2).normal(size=4096).astype(f32) * 100
    expect = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    assert_bit_exact(port.round_bf16(x), expect, "bf16 RNE")
    t = port.round_tf32(x)
    assert np.all((t.view(np.uint32) & 0x1fff) == 0)
    assert np.all(np.abs(t - x) <= np.abs(x) * 2.0 ** -11)


@needs_ref
def test_port_softmax_reduce_mean_match_reference_bits(rng):
    """softmax (last axis) and reduce_mean: the plain-C port against the kernels the reference's compiler generates.
    Both use the C library's expf and the same sequential sums, so the bits agree."""
    x = rng.normal(0, 2, (3, 5, 7)).astype(np.float32)
    assert_bit_exact(port.softmax(x, -1), ref.softmax(x, -1), "softmax last axis")
    assert_bit_exact(port.softmax(x.reshape(15, 7), 1), ref.softmax(x.reshape(15, 7), 1), "softmax rank 2")
    assert np.abs(port.softmax(x, 2).sum(2) - 1).max() < 1e-6
    for axes, keep in (((2,), True), ((1, 2), True), ((0, 2), False), ((1,), False), ((0,), False), ((0, 1, 2), True)):
        assert_bit_exact(port.reduce_mean(x, axes, keep), ref.reduce_mean(x, axes, keep), f"reduce_mean {axes} keepdims={keep}")
    # global average pooling is reduce_mean over (2, 3) with keepdims
    y = rng.normal(0, 1, (2, 3, 4, 5)).astype(np.float32)
    assert_bit_exact(port.reduce_mean(y, (2, 3), True), port.global_avg_pool2d(y), "reduce_mean == global_avg_pool2d")
    with pytest.raises(ValueError):
        port.softmax(x, 0)      # the reference's own result for an inner axis is not a softmax
    with pytest.raises(ValueError):
        port.reduce_mean(x, (0,), True)



@needs_ref
def test_port_matmul_transpose_reshape_cast_match_reference_bits(rng):
    """matmul, transpose, reshape and cast: the plain-C port against the kernels the reference's compiler generates.
    cast is compiled with the one-macro shim `cast(x) = (x)`: the reference's C backend prints the call but never
    defines it (src/codegen/codegen_c.cc:155-169); the assignment then converts like CodeGenLLVM::CastValue."""
    a = rng.normal(0, 1, (9, 13)).astype(np.float32)
    b = rng.normal(0, 1, (13, 6)).astype(np.float32)
    assert_bit_exact(port.matmul(a, b), ref.matmul(a, b), "matmul")
    x = rng.normal(0, 1, (2, 3, 4, 5)).astype(np.float32)
    for axes in (None, (0, 2, 3, 1), (0, 3, 1, 2), (3, 2, 1, 0), (1, 0, 2, 3), (0, 1, 3, 2), (-1, 0, 1, 2), (0, 1, 2, 3)):
        got = port.transpose(x, axes)
        assert_bit_exact(got, ref.transpose(x, axes), f"transpose {axes}")
        assert_bit_exact(got, np.ascontiguousarray(np.transpose(x, axes)), f"transpose {axes} vs numpy")
    xi = rng.integers(-1000, 1000, (7, 11)).astype(np.int32)
    assert_bit_exact(port.transpose(xi, (1, 0)), ref.transpose(xi, (1, 0)), "transpose int32")
    assert_bit_exact(ref.reshape(x, (0, -1, 5), (2, 12, 5)), port.reshape(x, (2, 12, 5)), "reshape 0/-1")
    assert_bit_exact(ref.reshape(x, (120,), (120,)), port.reshape(x, (120,)), "reshape flat")
    v = rng.normal(0, 40, (4, 9)).astype(np.float32)
    v[0, :4] = (0.0, -0.0, 0.999, -0.999)
    for dt in (np.int32, np.int64, np.float64, np.int8):
        assert_bit_exact(port.cast(v, dt), ref.cast(v, dt), f"cast float32 -> {np.dtype(dt).name}")
    assert_bit_exact(port.cast(np.abs(v), np.uint8), ref.cast(np.abs(v), np.uint8), "cast float32 -> uint8")
    big = np.array([2**31 - 1, -2**31, 16777217, -16777217, 300, -300, 127, -128, 255, 0], dtype=np.int32)
    for dt in (np.float32, np.int64, np.float64, np.int8, np.uint8):
        assert_bit_exact(port.cast(big, dt), ref.cast(big, dt), f"cast int32 -> {np.dtype(dt).name}")
    wide = np.array([2**40 + 5, -2**40 - 5, 2**53 + 1, -7, 2**31], dtype=np.int64)
    for dt in (np.float32, np.int32, np.float64):
        assert_bit_exact(port.cast(wide, dt), ref.cast(wide, dt), f"cast int64 -> {np.dtype(dt).name}")
    d = np.array([1.0 + 2.0**-30, -3.999999, 1e-50, 123456.789, 0.1], dtype=np.float64)
    for dt in (np.float32, np.int32, np.int64):
        assert_bit_exact(port.cast(d, dt), ref.cast(d, dt), f"cast float64 -> {np.dtype(dt).name}")
    s8 = np.array([-128, -1, 0, 1, 127], dtype=np.int8)
    u8 = np.array([0, 1, 127, 128, 255], dtype=np.uint8)
    for dt in (np.float32, np.int32, np.int64, np.uint8):
        assert_bit_exact(port.cast(s8, dt), ref.cast(s8, dt), f"cast int8 -> {np.dtype(dt).name}")
    for dt in (np.float32, np.int32, np.int64, np.int8):
        assert_bit_exact(port.cast(u8, dt), ref.cast(u8, dt), f"cast uint8 -> {np.dtype(dt).name}")

"""ResNet-18 as the reference builds it (test/resnet18_ir_dump.cpp:191-452): 49 Relay calls —
20 nn_conv2d (BatchNorm already folded into weight + bias), 17 nn_relu, 8 add, nn_max_pool2d,
nn_global_avg_pool2d, nn_flatten, nn_gemm(alpha=1, beta=1, transB=1) — with seed-generated weights.

The reference's resnet18.onnx is not part of its repository, so weights follow the benchmark
configuration instead: Kaiming-normal convolutions, BatchNorm gamma~U(0.5,1.5), beta~N(0,0.1),
mean~N(0,0.1), var~U(0.5,1.5) folded on the host in fp32 with eps=1e-5 (BatchNormAttrs default,
include/relay/op.h:196): W' = W*g/sqrt(v+eps), b' = beta - mean*g/sqrt(v+eps).
"""
import numpy as np

from . import relay

# (name, cin, cout, k, stride, pad) in the reference's node order; "ds" = 1x1 stride-2 downsample
_STAGES = [(64, 1), (128, 2), (256, 2), (512, 2)]


def make_weights(seed=0, num_classes=1000):
    """Returns a list of (name, np.float32 array) in creation order: conv weight/bias pairs, fc.weight, fc.bias."""
    rng = np.random.default_rng(seed)
    out = []

    def conv_bn(name, cin, cout, k):
        w = rng.normal(0.0, np.sqrt(2.0 / (cin * k * k)), (cout, cin, k, k)).astype(np.float32)
        gamma = rng.uniform(0.5, 1.5, cout).astype(np.float32)
        beta = rng.normal(0.0, 0.1, cout).astype(np.float32)
        mean = rng.normal(0.0, 0.1, cout).astype(np.float32)
        var = rng.uniform(0.5, 1.5, cout).astype(np.float32)
        scale = (gamma / np.sqrt(var + np.float32(1e-5))).astype(np.float32)
        out.append((name + ".weight", (w * scale[:, None, None, None]).astype(np.float32)))
        out.append((name + ".bias", (beta - mean * scale).astype(np.float32)))

    conv_bn("conv1", 3, 64, 7)
    cin = 64
    for si, (cout, stride) in enumerate(_STAGES, start=1):
        for bi in range(2):
            s = stride if bi == 0 else 1
            conv_bn(f"layer{si}.{bi}.conv1", cin, cout, 3)
            conv_bn(f"layer{si}.{bi}.conv2", cout, cout, 3)
            if s != 1 or cin != cout:
                conv_bn(f"layer{si}.{bi}.downsample", cin, cout, 1)
            cin = cout
    out.append(("fc.weight", rng.normal(0.0, np.sqrt(2.0 / 512), (num_classes, 512)).astype(np.float32)))
    out.append(("fc.bias", rng.normal(0.0, 0.01, num_classes).astype(np.float32)))
    return out


def build(batch, weights, to_constant=lambda a: a):
    """Relay function for a given batch size. `weights` as from make_weights(); `to_constant` maps a
    numpy array to the object stored in Constant.data (e.g. a CUDA tensor)."""
    w = {name: relay.Constant(to_constant(arr), name) for name, arr in weights}
    x = relay.Var("input", (batch, 3, 224, 224))

    def conv(data, name, stride, pad):
        return relay.Call("nn_conv2d", [data, w[name + ".weight"], w[name + ".bias"]],
                          relay.Conv2DAttrs((stride, stride), (pad, pad, pad, pad), (1, 1), 1))

    def relu(e):
        return relay.Call("nn_relu", [e])

    y = relu(conv(x, "conv1", 2, 3))
    y = relay.Call("nn_max_pool2d", [y], relay.MaxPool2DAttrs((2, 2), (1, 1, 1, 1), (1, 1), (3, 3), "NCHW", False))
    cin = 64
    for si, (cout, stride) in enumerate(_STAGES, start=1):
        for bi in range(2):
            s = stride if bi == 0 else 1
            name = f"layer{si}.{bi}"
            a = relu(conv(y, name + ".conv1", s, 1))
            b = conv(a, name + ".conv2", 1, 1)
            identity = conv(y, name + ".downsample", s, 0) if (name + ".downsample.weight") in w else y
            y = relu(relay.Call("add", [b, identity]))
            cin = cout
    y = relay.Call("nn_global_avg_pool2d", [y])
    y = relay.Call("nn_flatten", [y])
    y = relay.Call("nn_gemm", [y, w["fc.weight"], w["fc.bias"]], relay.GemmAttrs(1.0, 1.0, 0, 1))
    return relay.Function([x], y)


# The 11 distinct convolution shapes: (name, cin, cout, k, stride, pad, input H=W, count in the network)
CONV_SHAPES = [
    ("stem", 3, 64, 7, 2, 3, 224, 1), ("l1", 64, 64, 3, 1, 1, 56, 4), ("l2a", 64, 128, 3, 2, 1, 56, 1),
    ("l2", 128, 128, 3, 1, 1, 28, 3), ("l2ds", 64, 128, 1, 2, 0, 56, 1), ("l3a", 128, 256, 3, 2, 1, 28, 1),
    ("l3", 256, 256, 3, 1, 1, 14, 3), ("l3ds", 128, 256, 1, 2, 0, 28, 1), ("l4a", 256, 512, 3, 2, 1, 14, 1),
    ("l4", 512, 512, 3, 1, 1, 7, 3), ("l4ds", 256, 512, 1, 2, 0, 14, 1),
]


def conv_flops_per_image():
    """2*Cout*OH*OW*Cin*KH*KW summed over the 20 convolutions (padded taps counted)."""
    total = 0
    for _, cin, cout, k, s, p, h, count in CONV_SHAPES:
        oh = (h + 2 * p - k) // s + 1
        total += count * 2 * cout * oh * oh * cin * k * k
    return total


FC_FLOPS_PER_IMAGE = 2 * 512 * 1000

"""Layer table of the ResNet-50 (v1.5: stride on the 3x3) convolution stack, and of one stage-3
bottleneck block: the workloads the reference's layer benchmark is built around
(`Conv2dProblem` presets, src/optimizer/benchmark.rs:474-509; examples/resnet_bench.rs:28-47).
BatchNorm is folded into a per-channel bias, ReLU / residual are fused into the conv epilogue; the
max-pool after the stem and the FC head are not convolutions and are not part of the stack.
"""
from collections import namedtuple

# src: name of the tensor the conv reads; res: name of the tensor added before the activation
ConvSpec = namedtuple("ConvSpec", "name src res dst C H W K R S stride pad epilogue")


def out_hw(h, r, stride, pad):
    return (h + 2 * pad - r) // stride + 1


def bottleneck(prefix, src, cin, h, width, stride, downsample):
    """The 3 (or 4, with a projection shortcut) convs of one bottleneck block reading tensor `src`."""
    cout = 4 * width
    ho = out_hw(h, 3, stride, 1)
    specs = []
    res = src
    if downsample:
        specs.append(ConvSpec(prefix + ".ds", src, None, prefix + ".ds", cin, h, h, cout, 1, 1, stride, 0, "bias"))
        res = prefix + ".ds"
    specs.append(ConvSpec(prefix + ".c1", src, None, prefix + ".c1", cin, h, h, width, 1, 1, 1, 0, "bias+relu"))
    specs.append(ConvSpec(prefix + ".c2", prefix + ".c1", None, prefix + ".c2", width, h, h, width, 3, 3, stride, 1,
                          "bias+relu"))
    specs.append(ConvSpec(prefix + ".c3", prefix + ".c2", res, prefix + ".out", width, ho, ho, cout, 1, 1, 1, 0,
                          "bias+residual+relu"))
    return specs, prefix + ".out", cout, ho


def resnet50_convs():
    """All 53 convolutions. Two tensors are inputs of the stack: 'image' (N,3,224,224) for the stem
    and 'pooled' (N,64,56,56) for layer1 -- the max-pool between them is not a convolution, so
    layer1 reads a separate synthetic tensor of the pooled shape instead."""
    specs = [ConvSpec("stem", "image", None, "stem", 3, 224, 224, 64, 7, 7, 2, 3, "bias+relu")]
    src, cin, h = "pooled", 64, 56
    for stage, (width, blocks) in enumerate(((64, 3), (128, 4), (256, 6), (512, 3)), start=1):
        for b in range(blocks):
            stride = 2 if (b == 0 and stage > 1) else 1
            blk, src, cin, h = bottleneck("layer%d.%d" % (stage, b), src, cin, h, width, stride, b == 0)
            specs.extend(blk)
    return specs


def stage3_bottleneck():
    """One identity-shortcut bottleneck block of stage 3: 1x1 1024->256, 3x3 256->256, 1x1 256->1024
    with the block input added before the last ReLU, on 14x14 feature maps."""
    specs, _, _, _ = bottleneck("block", "input", 1024, 14, 256, 1, False)
    return specs


def conv_flops(spec, n):
    """2 * M * Ngemm * Kgemm, the reference's convention (src/optimizer/benchmark.rs:458-469):
    padding taps counted, epilogue not counted."""
    ho, wo = out_hw(spec.H, spec.R, spec.stride, spec.pad), out_hw(spec.W, spec.S, spec.stride, spec.pad)
    return 2.0 * n * ho * wo * spec.K * spec.C * spec.R * spec.S


def conv_bytes(spec, n, elem_size=2):
    """Algorithmic bytes: every tensor touched once (a strided 1x1 conv only reads the pixels it
    samples); bias as fp32."""
    ho, wo = out_hw(spec.H, spec.R, spec.stride, spec.pad), out_hw(spec.W, spec.S, spec.stride, spec.pad)
    in_px = ho * wo if (spec.R == 1 and spec.S == 1) else spec.H * spec.W
    b = n * in_px * spec.C * elem_size + spec.K * spec.C * spec.R * spec.S * elem_size + n * ho * wo * spec.K * elem_size
    b += spec.K * 4
    if spec.res is not None:
        b += n * ho * wo * spec.K * elem_size
    return float(b)

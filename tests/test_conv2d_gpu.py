"""Parity of the CUDA path against the CPU oracle, through the C ABI, on a B200.

Tolerances (written here once, used everywhere below):
  fp16 / bf16 inputs, fp32 accumulation:  max|out - ref| <= 1e-2 * max|ref|
  fp32 inputs computed as TF32:           max|out - ref| <= 5e-3 * max|ref|
The oracle is fed the inputs already rounded to the storage type, accumulates in fp32 and is rounded
to the storage type once at the end, like the kernel's single rounding after the epilogue.
"""
import os

import numpy as np
import pytest
import torch

import convcases as cc
from golden.make_golden import CASES
from oracle import oracle
from tracea_b200 import ffi, ops, resnet50, runner

pytestmark = pytest.mark.gpu

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "conv2d_golden.npz"))
TORCH_DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def to_dev(a, dtype, channels_last=True):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(TORCH_DT[dtype]).cuda()
    if channels_last and t.ndim == 4:
        t = t.contiguous(memory_format=torch.channels_last)
    return t


def split_epi(epi):
    ops_ = [o for o in (epi or "").split("+") if o]
    act = next((o for o in ops_ if o in ("relu", "silu", "gelu")), "none")
    return "bias" in ops_, "residual" in ops_, act


def run_gpu(x, w, b, res, stride, padding, dilation, epi, dtype, channels_last=True, out_channels_last=None):
    use_b, use_r, _ = split_epi(epi)
    tx, tw = to_dev(x, dtype, channels_last), to_dev(w, dtype, channels_last)
    tb = torch.from_numpy(b).cuda() if use_b else None
    tr = to_dev(res, dtype, channels_last if out_channels_last is None else out_channels_last) if use_r else None
    out = ops.conv2d_nchw(tx, tw, tb, tr, stride, padding, dilation, 1, epi or None,
                          channels_last_out=out_channels_last)
    torch.cuda.synchronize()
    assert ffi.load().tracea_b200_device_status(0) == 0
    return out.float().cpu().numpy()


def run_oracle(x, w, b, res, stride, padding, dilation, epi, dtype, fast=True):
    use_b, use_r, act = split_epi(epi)
    xr, wr = cc.round_to(x, dtype), cc.round_to(w, dtype)
    rr = cc.round_to(res, dtype) if use_r else None
    if fast:
        out = oracle.conv2d_gemm(cc.channels_last(xr), wr, b if use_b else None, rr, stride, padding, dilation, act)
    else:
        out = oracle.conv2d(xr, wr, b if use_b else None, rr, stride, padding, dilation, act)
    return cc.round_to(np.ascontiguousarray(out), dtype)


def check(x, w, b, res, stride, padding, dilation, epi, dtype, **kw):
    got = run_gpu(x, w, b, res, stride, padding, dilation, epi, dtype, **kw)
    want = run_oracle(x, w, b, res, stride, padding, dilation, epi, dtype)
    assert got.shape == want.shape
    err = cc.rel_err(got, want)
    assert err <= cc.tol_for(dtype), "rel err %.3g" % err
    return got, want


# --------------------------------------------------------------------------- golden fixtures
@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_golden_fixtures(name, dtype):
    spec = CASES[name]
    x, w, b, res, ref = (GOLDEN[name + "/" + k] for k in ("x", "w", "b", "res", "out"))
    got, _ = check(x, w, b, res, spec[7], spec[8], spec[9], spec[10], dtype)
    if dtype == "f32":   # also directly against the committed fp32 known answers
        assert cc.rel_err(got, ref) <= cc.TOL_TF32


@pytest.mark.parametrize("name", ["verify_conv2d_rs", "bias_relu_3x3", "stem_7x7_s2_c3", "dilated_asym"])
def test_golden_fixtures_from_nchw_memory(name):
    """NCHW-contiguous x / OIHW-contiguous w (the layout include/tracea.hpp documents) and NCHW out."""
    spec = CASES[name]
    x, w, b, res, ref = (GOLDEN[name + "/" + k] for k in ("x", "w", "b", "res", "out"))
    got, _ = check(x, w, b, res, spec[7], spec[8], spec[9], spec[10], "f32", channels_last=False,
                   out_channels_last=False)
    assert cc.rel_err(got, ref) <= cc.TOL_TF32


# --------------------------------------------------------------------------- the five benchmark configs
def test_config1_fp32_nchw_full():
    x = cc.uniform((1, 64, 56, 56), 0, "cfg1/x")
    w = cc.uniform((64, 64, 3, 3), 0, "cfg1/w")
    b = cc.normal((64,), 0, "cfg1/b", 0.1)
    got = run_gpu(x, w, b, None, 1, 1, 1, "bias+relu", "f32", channels_last=False, out_channels_last=False)
    want = oracle.conv2d(x, w, b, None, 1, 1, 1, "relu")          # the scalar restatement, full size
    assert cc.rel_err(got, want) <= cc.TOL_TF32
    dig = np.load(os.path.join(os.path.dirname(__file__), "golden", "conv2d_cfg1_digest.npz"))
    assert np.abs(got.reshape(-1)[::7] - dig["out_every7"]).max() <= cc.TOL_TF32 * float(dig["out_absmax"][0])


def test_config2_fp16_readme_shape_full():
    x = cc.uniform((1, 64, 224, 224), 0, "cfg2/x")
    w = cc.kaiming((128, 64, 3, 3), 0, "cfg2/w")
    got, want = check(x, w, None, None, 1, 0, 1, "", "f16", channels_last=False, out_channels_last=False)
    assert got.shape == (1, 128, 222, 222)      # M = 49284 is not a multiple of the 128-pixel tile


def _block_inputs(n):
    x = np.abs(cc.normal((n, 1024, 14, 14), 0, "cfg3/x"))
    ws = [cc.kaiming((256, 1024, 1, 1), 0, "cfg3/w1"), cc.kaiming((256, 256, 3, 3), 0, "cfg3/w2"),
          cc.kaiming((1024, 256, 1, 1), 0, "cfg3/w3")]
    bs = [cc.normal((k,), 0, "cfg3/b%d" % i, 0.05) for i, k in enumerate((256, 256, 1024))]
    return x, ws, bs


def _block_oracle(x, ws, bs):
    """Chained oracle: each layer's output is rounded to bf16 before it feeds the next one."""
    xr = cc.round_to(x, "bf16")
    y1 = run_oracle(xr, ws[0], bs[0], None, 1, 0, 1, "bias+relu", "bf16")
    y2 = run_oracle(y1, ws[1], bs[1], None, 1, 1, 1, "bias+relu", "bf16")
    y3 = run_oracle(y2, ws[2], bs[2], xr, 1, 0, 1, "bias+residual+relu", "bf16")
    return y1, y2, y3


def _block_gpu(x, ws, bs):
    n = x.shape[0]
    specs = resnet50.stage3_bottleneck()
    weights = {sp.name: (torch.from_numpy(w), torch.from_numpy(b)) for sp, w, b in zip(specs, ws, bs)}
    stack = runner.ConvStack(specs, n, "bf16", "cuda", inputs={"input": to_dev(x, "bf16")}, weights=weights)
    stack.forward()
    torch.cuda.synchronize()
    assert ffi.load().tracea_b200_device_status(0) == 0
    return stack


def test_config3_bottleneck_block_chain_n8_full_tensors():
    x, ws, bs = _block_inputs(8)
    stack = _block_gpu(x, ws, bs)
    y1, y2, y3 = _block_oracle(x, ws, bs)
    for name, want in (("block.c1", y1), ("block.c2", y2), ("block.out", y3)):
        got = stack.tensors[name].float().cpu().numpy()
        assert cc.rel_err(got, want) <= cc.TOL_16BIT, name


def test_config3_bottleneck_block_n256_sampled_and_shard_invariant():
    """Full batch: 2*10^4 output points per layer against fp64 dot products of that layer's actual
    (GPU-produced, bf16) input, and bit-exact agreement of images 0..7 with the N=8 run."""
    x, ws, bs = _block_inputs(256)
    stack = _block_gpu(x, ws, bs)
    small = _block_gpu(x[:8], ws, bs)
    for name in ("block.c1", "block.c2", "block.out"):
        assert torch.equal(stack.tensors[name][:8], small.tensors[name]), name
    rng = np.random.default_rng(3)
    xin = stack.tensors["input"].float().cpu().numpy()
    y1 = stack.tensors["block.c1"].float().cpu().numpy()
    y2 = stack.tensors["block.c2"].float().cpu().numpy()
    y3 = stack.tensors["block.out"].float().cpu().numpy()
    layers = [(xin, ws[0], bs[0], None, 0, "relu", y1), (y1, ws[1], bs[1], None, 1, "relu", y2),
              (y2, ws[2], bs[2], xin, 0, "relu", y3)]
    for src, w, b, res, pad, act, got in layers:
        idx = np.stack([rng.integers(0, s, 20000) for s in got.shape], axis=1)
        want = oracle.conv2d_points(src, cc.round_to(w, "bf16"), idx, b, res, 1, pad, 1, act, acc_double=True)
        vals = got[idx[:, 0], idx[:, 1], idx[:, 2], idx[:, 3]]
        assert np.abs(vals - want).max() <= cc.TOL_16BIT * np.abs(want).max()


def test_config4_strided_downsample_bias_silu():
    # full N = 256 on the GPU; images 0..3 against the oracle in full, 2*10^4 points over the rest
    n = 256
    x = cc.normal((n, 128, 56, 56), 0, "cfg4/x")
    w = cc.kaiming((256, 128, 3, 3), 0, "cfg4/w")
    b = cc.normal((256,), 0, "cfg4/b", 0.1)
    got = run_gpu(x, w, b, None, 2, 1, 1, "bias+silu", "bf16")
    assert got.shape == (n, 256, 28, 28)
    want4 = run_oracle(x[:4], w, b, None, 2, 1, 1, "bias+silu", "bf16")
    assert cc.rel_err(got[:4], want4) <= cc.TOL_16BIT
    rng = np.random.default_rng(4)
    idx = np.stack([rng.integers(0, s, 20000) for s in got.shape], axis=1)
    want = oracle.conv2d_points(cc.round_to(x, "bf16"), cc.round_to(w, "bf16"), idx, b, None, 2, 1, 1, "silu")
    vals = got[idx[:, 0], idx[:, 1], idx[:, 2], idx[:, 3]]
    assert np.abs(vals - want).max() <= cc.TOL_16BIT * np.abs(want).max()


def _stack_inputs(n):
    img = cc.normal((n, 3, 224, 224), 0, "cfg5/image")    # a true 3-channel image
    pooled = np.abs(cc.normal((n, 64, 56, 56), 0, "cfg5/pooled"))
    return img, pooled


def test_config5_resnet50_conv_stack_n2_every_layer():
    """All 53 convs at N=2: every layer's output against the oracle applied to that layer's actual
    (GPU-produced) input, so one wrong layer cannot hide behind another."""
    n = 2
    img, pooled = _stack_inputs(n)
    specs = resnet50.resnet50_convs()
    stack = runner.ConvStack(specs, n, "bf16", "cuda", seed=5,
                             inputs={"image": to_dev(img, "bf16"), "pooled": to_dev(pooled, "bf16")})
    stack.forward()
    torch.cuda.synchronize()
    assert ffi.load().tracea_b200_device_status(0) == 0
    for sp in specs:
        src = stack.tensors[sp.src].float().cpu().numpy()
        w = stack.weights[sp.name].float().cpu().numpy()
        b = stack.biases[sp.name].cpu().numpy()
        res = stack.tensors[sp.res].float().cpu().numpy() if sp.res is not None else None
        _, _, act = split_epi(sp.epilogue)
        want = oracle.conv2d_gemm(cc.channels_last(src), w, b, res, sp.stride, sp.pad, 1, act)
        got = stack.tensors[sp.dst].float().cpu().numpy()
        assert cc.rel_err(got, cc.round_to(np.ascontiguousarray(want), "bf16")) <= cc.TOL_16BIT, sp.name


def _sampled_layer_check(stack, sp, images, points, rng):
    """One layer of a resident conv stack against fp64 dot products over its actual (GPU-produced) input, on
    `points` output points spread over the images `images` (a convolution never mixes images, so the sub-batch is
    checked as a batch of its own)."""
    sel = torch.as_tensor(images, device="cuda")
    src = stack.tensors[sp.src].index_select(0, sel).float().cpu().numpy()
    got = stack.tensors[sp.dst].index_select(0, sel).float().cpu().numpy()
    res = stack.tensors[sp.res].index_select(0, sel).float().cpu().numpy() if sp.res is not None else None
    w = stack.weights[sp.name].float().cpu().numpy()
    b = stack.biases[sp.name].cpu().numpy()
    _, _, act = split_epi(sp.epilogue)
    idx = np.stack([rng.integers(0, s, points) for s in got.shape], axis=1)
    want = oracle.conv2d_points(src, w, idx, b, res, sp.stride, sp.pad, 1, act, acc_double=True)
    vals = got[idx[:, 0], idx[:, 1], idx[:, 2], idx[:, 3]]
    assert np.abs(vals - want).max() <= cc.TOL_16BIT * np.abs(want).max(), sp.name


@pytest.mark.parametrize("n", [64, 512])
def test_config5_resnet50_conv_stack_at_the_benchmark_batches(n):
    """The 53 convs at the per-GPU batches the benchmark times them at (512 on one GPU, 64 on each of eight):
    here every layer runs its multi-wave, panelled and CTA-pair tilings. Each layer: 2*10^4 output points
    over eight images (the first, the last, six in between) against the oracle on the layer's own input; and
    images 0..1 of every tensor against the N=2 run of the same stack (the ResNet-50 layer shapes of
    src/optimizer/benchmark.rs:474-509 at full batch)."""
    img, pooled = _stack_inputs(8)
    reps = (n + 7) // 8
    specs = resnet50.resnet50_convs()

    def make(count):
        ti = to_dev(img, "bf16").repeat(reps, 1, 1, 1)[:count].contiguous(memory_format=torch.channels_last)
        tp = to_dev(pooled, "bf16").repeat(reps, 1, 1, 1)[:count].contiguous(memory_format=torch.channels_last)
        # images differ across the batch: scale image i by a power of two (exact in bf16)
        scale = (2.0 ** (torch.arange(count, device="cuda") % 3 - 1)).to(torch.bfloat16).view(-1, 1, 1, 1)
        cl = lambda t: t.contiguous(memory_format=torch.channels_last)
        return runner.ConvStack(specs, count, "bf16", "cuda", seed=5,
                                inputs={"image": cl(ti * scale), "pooled": cl(tp * scale)})

    stack = make(n)
    stack.forward()
    torch.cuda.synchronize()
    assert ffi.load().tracea_b200_device_status(0) == 0
    rng = np.random.default_rng(50 + n)
    for sp in specs:
        images = sorted({0, n - 1, *rng.integers(1, n - 1, 6).tolist()})
        _sampled_layer_check(stack, sp, images, 20000, rng)
    small = make(2)
    small.forward()
    torch.cuda.synchronize()
    for sp in specs:   # every tile accumulates over K in the same order whatever the batch size: identical bits
        assert torch.equal(stack.tensors[sp.dst][:2], small.tensors[sp.dst]), sp.name


def test_config3_c2_n256_full_tensor_against_the_oracle():
    """The headline layer (3x3 256->256 at 256 images) compared in full: all 12.8 M outputs against the oracle's
    im2col + GEMM path on the layer's actual bf16 input."""
    x, ws, bs = _block_inputs(256)
    stack = _block_gpu(x, ws, bs)
    y1 = stack.tensors["block.c1"].float().cpu().numpy()
    want = oracle.conv2d_gemm(cc.channels_last(y1), cc.round_to(ws[1], "bf16"), bs[1], None, 1, 1, 1, "relu")
    got = stack.tensors["block.c2"].float().cpu().numpy()
    assert cc.rel_err(got, cc.round_to(np.ascontiguousarray(want), "bf16")) <= cc.TOL_16BIT


# --------------------------------------------------------------------------- size-independent properties
def test_identity_filter_reproduces_the_input_bit_exactly_at_full_size():
    """A 1x1 filter that is the identity matrix copies x to out exactly (x*1 + 0*... in fp32 is
    exact), which checks every (pixel, channel) address of a full-size tensor."""
    n, c = 256, 256
    x = to_dev(cc.normal((n, c, 14, 14), 0, "prop/x"), "bf16")
    w = torch.eye(c, dtype=torch.bfloat16, device="cuda").view(c, c, 1, 1).contiguous(memory_format=torch.channels_last)
    out = ops.conv2d_nchw(x, w)
    assert torch.equal(out, x)


def test_shifted_delta_filter_is_an_exact_shift_with_zero_padding():
    n, c, h = 64, 64, 28
    x = to_dev(cc.normal((n, c, h, h), 0, "prop/x2"), "bf16")
    for (r, s) in ((0, 0), (1, 2), (2, 1)):
        w = torch.zeros(c, c, 3, 3, device="cuda")
        w[torch.arange(c), torch.arange(c), r, s] = 1.0
        w = w.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        out = ops.conv2d_nchw(x, w, padding=1)
        want = torch.zeros_like(x)
        dh, dw = r - 1, s - 1
        hs, ws_ = slice(max(0, -dh), h - max(0, dh)), slice(max(0, -dw), h - max(0, dw))
        hd, wd = slice(max(0, dh), h + min(0, dh)), slice(max(0, dw), h + min(0, dw))
        want[:, :, hs, ws_] = x[:, :, hd, wd]
        assert torch.equal(out, want), (r, s)


def test_zero_weights_give_activation_of_bias():
    x = to_dev(cc.normal((4, 64, 9, 9), 0, "prop/x3"), "bf16")
    w = torch.zeros(96, 64, 3, 3, dtype=torch.bfloat16, device="cuda").contiguous(memory_format=torch.channels_last)
    b = torch.from_numpy(cc.normal((96,), 0, "prop/b3")).cuda()
    out = ops.conv2d_nchw(x, w, b, padding=1, epilogue="bias+relu")
    want = torch.relu(b).to(torch.bfloat16).view(1, -1, 1, 1).expand_as(out)
    assert torch.equal(out, want)


def test_batch_shards_concatenate_to_the_full_batch_bit_exactly():
    from tracea_b200 import shard
    n = 37
    x = to_dev(cc.normal((n, 64, 14, 14), 0, "prop/x4"), "bf16")
    w = to_dev(cc.kaiming((128, 64, 3, 3), 0, "prop/w4"), "bf16")
    b = torch.from_numpy(cc.normal((128,), 0, "prop/b4", 0.1)).cuda()
    full = ops.conv2d_nchw(x, w, b, padding=1, epilogue="bias+silu")
    for world in (2, 4, 8):
        parts = []
        for r in range(world):
            a, e = shard.shard_range(n, r, world)
            parts.append(ops.conv2d_nchw(x[a:e], w, b, padding=1, epilogue="bias+silu"))
        assert torch.equal(torch.cat(parts), full), world


# --------------------------------------------------------------------------- edge cases
EDGE = [
    # N, C, H, W, K, R, S, stride, pad, dil, epi
    (1, 64, 1, 1, 64, 1, 1, 1, 0, 1, ""),                  # single pixel
    (1, 8, 2, 2, 8, 3, 3, 1, 1, 1, "bias"),                # filter larger than the image, kept by padding
    (3, 64, 15, 15, 64, 3, 3, 1, 1, 1, "bias+relu"),       # M = 675: ragged last tile
    (1, 64, 16, 16, 72, 3, 3, 1, 1, 1, "bias+relu"),       # K_out tail inside a tile
    (1, 64, 16, 16, 66, 3, 3, 1, 1, 1, "bias+relu"),       # K_out not a multiple of 8: scalar stores
    (2, 3, 17, 19, 5, 3, 3, 1, 1, 1, "bias+relu"),         # C = 3: channel-padding adapter
    (2, 20, 9, 9, 300, 1, 1, 1, 0, 1, "bias"),             # C = 20 (padded to 24), K_out > 256
    (2, 96, 10, 10, 64, 3, 3, 1, 1, 1, ""),                # 192-byte pixels: 64-byte k-chunks
    (2, 16, 10, 10, 64, 3, 3, 1, 1, 1, ""),                # 32-byte k-chunks
    (2, 8, 10, 10, 64, 5, 5, 1, 2, 1, ""),                 # 16-byte k-chunks, odd chunk count
    (1, 64, 40, 40, 32, 3, 3, (2, 1), (0, 1), 1, "silu"),  # different stride / padding per axis
    (1, 32, 23, 23, 32, 3, 3, 3, 4, 2, "gelu"),            # stride 3, large padding, dilation 2
    (1, 64, 32, 32, 64, 7, 7, 2, 3, 1, "bias+relu"),       # 7x7 / 2
    (5, 64, 7, 7, 2048, 1, 1, 1, 0, 1, "bias+relu"),       # wide output, tiny image
    (2, 3, 37, 41, 64, 7, 7, 2, 3, 1, "bias+relu"),        # RGB stem: filter rows fetched as windows (16-bit: 8-byte
                                                           # pixels, odd padded width; fp32: 16-byte pixels)
    (2, 4, 20, 30, 16, 2, 8, (1, 2), (0, 3), 1, ""),       # 8-byte pixels, 8-wide filter row fills the whole window
    (1, 2, 15, 40, 24, 3, 4, (1, 4), (1, 2), 1, "bias"),   # 8-byte pixels, horizontal stride 4 (two W units a step)
    (2, 1, 30, 30, 8, 5, 5, 2, 2, 1, "relu"),              # single-channel image, 5x5 / 2
    (1, 3, 64, 300, 32, 3, 3, 2, 1, 1, "bias+relu"),       # 8-byte pixels, rows wider than one tile
    (2, 8, 20, 30, 16, 2, 8, (1, 2), (0, 3), 1, ""),       # 8-wide filter row fills the whole window
    (2, 8, 20, 30, 16, 3, 9, 1, (1, 4), 1, ""),            # 9-wide filter: too wide for a window, per-tap path
    (2, 8, 21, 21, 16, 3, 3, 1, 2, (1, 2), "silu"),        # 16-byte pixels with horizontal dilation: per-tap path
    (1, 4, 9, 200, 8, 1, 5, 1, (0, 2), 1, "bias"),         # one-row filter on a wide image
]


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("case", EDGE, ids=lambda c: "N%dC%dH%dW%dK%dR%dS%d" % c[:7])
def test_edge_cases(case, dtype):
    N, C, H, W, K, R, S, stride, pad, dil, epi = case
    x = cc.uniform((N, C, H, W), 1, "edge/x")
    w = cc.kaiming((K, C, R, S), 1, "edge/w")
    b = cc.normal((K,), 1, "edge/b", 0.1)
    ho, wo = oracle.out_shape(x.shape, w.shape, stride, pad, dil)[2:]
    res = cc.normal((N, K, ho, wo), 1, "edge/res")
    check(x, w, b, res, stride, pad, dil, epi, dtype)


@pytest.mark.parametrize("kind,use_bias,use_res,act", [
    (ffi.EPILOGUE_IDENTITY, False, False, "none"),
    (ffi.EPILOGUE_BIAS_ADD, True, False, "none"),
    (ffi.EPILOGUE_RELU, False, False, "relu"),       # a bias handed to a non-BIAS kind is ignored,
    (ffi.EPILOGUE_GELU, False, False, "gelu"),       # as in src/interface/c_bindings.rs:144-197
    (ffi.EPILOGUE_SILU, False, False, "silu"),
    (ffi.EPILOGUE_BIAS_RELU, True, False, "relu"),
    (ffi.EPILOGUE_BIAS_SILU, True, False, "silu"),
    (ffi.EPILOGUE_RESIDUAL, False, True, "none"),
    (ffi.EPILOGUE_RESIDUAL_RELU, False, True, "relu"),
    (ffi.EPILOGUE_BIAS_RESIDUAL_RELU, True, True, "relu"),
    (ffi.EPILOGUE_BIAS_RESIDUAL, True, True, "none"),
])
def test_every_epilogue_kind_with_bias_and_residual_both_passed(kind, use_bias, use_res, act):
    x = cc.uniform((2, 64, 12, 12), 2, "epi/x")
    w = cc.kaiming((64, 64, 3, 3), 2, "epi/w")
    b = cc.normal((64,), 2, "epi/b", 0.5)
    res = cc.normal((2, 64, 12, 12), 2, "epi/res")
    out = ops.conv2d_nchw(to_dev(x, "bf16"), to_dev(w, "bf16"), torch.from_numpy(b).cuda(), to_dev(res, "bf16"),
                          1, 1, 1, 1, kind)
    want = oracle.conv2d_gemm(cc.channels_last(cc.round_to(x, "bf16")), cc.round_to(w, "bf16"),
                              b if use_bias else None, cc.round_to(res, "bf16") if use_res else None, 1, 1, 1, act)
    assert cc.rel_err(out.float().cpu().numpy(), cc.round_to(np.ascontiguousarray(want), "bf16")) <= cc.TOL_16BIT


def test_bias_silu_kind_without_bias_is_identity():
    # the reference emits the fused BiasAddSiLU op only when a bias tensor is present
    x = cc.uniform((1, 64, 8, 8), 2, "epi2/x")
    w = cc.kaiming((64, 64, 1, 1), 2, "epi2/w")
    out = ops.conv2d_nchw(to_dev(x, "bf16"), to_dev(w, "bf16"), None, None, 1, 0, 1, 1, ffi.EPILOGUE_BIAS_SILU)
    want = oracle.conv2d_gemm(cc.channels_last(cc.round_to(x, "bf16")), cc.round_to(w, "bf16"))
    assert cc.rel_err(out.float().cpu().numpy(), cc.round_to(np.ascontiguousarray(want), "bf16")) <= cc.TOL_16BIT


def test_bias_in_the_storage_dtype():
    x = cc.uniform((1, 64, 8, 8), 2, "bdt/x")
    w = cc.kaiming((64, 64, 3, 3), 2, "bdt/w")
    b = cc.normal((64,), 2, "bdt/b", 0.5)
    out = ops.conv2d_nchw(to_dev(x, "f16"), to_dev(w, "f16"), torch.from_numpy(b).half().cuda(), None, 1, 1, 1, 1,
                          "bias")
    want = oracle.conv2d_gemm(cc.channels_last(cc.round_to(x, "f16")), cc.round_to(w, "f16"), cc.round_to(b, "f16"),
                              None, 1, 1)
    assert cc.rel_err(out.float().cpu().numpy(), want) <= cc.TOL_16BIT


def test_ops_conv2d_nhwc_krsc_surface():
    """tracea.ops.conv2d: NHWC x, KRSC w, NHWK out (tracea-python/python/tracea/ops.py:39-70)."""
    x = cc.uniform((2, 64, 10, 12), 3, "ops/x")
    w = cc.kaiming((32, 64, 3, 3), 3, "ops/w")
    b = cc.normal((32,), 3, "ops/b", 0.1)
    x_nhwc = torch.from_numpy(x).permute(0, 2, 3, 1).contiguous().half().cuda()
    w_krsc = torch.from_numpy(w).permute(0, 2, 3, 1).contiguous().half().cuda()
    res = cc.normal((2, 10, 12, 32), 3, "ops/res")
    out = ops.conv2d(x_nhwc, w_krsc, bias=torch.from_numpy(b).cuda(), residual=torch.from_numpy(res).half().cuda(),
                     epilogue="bias+residual+relu", stride=1, padding=1)
    assert tuple(out.shape) == (2, 10, 12, 32)
    want = run_oracle(x, w, b, res.transpose(0, 3, 1, 2), 1, 1, 1, "bias+residual+relu", "f16")
    assert cc.rel_err(out.float().cpu().numpy().transpose(0, 3, 1, 2), want) <= cc.TOL_16BIT


def test_strided_output_view_leaves_the_gaps_alone():
    """out is a channel slice of a wider NHWC buffer (row pitch 96, K = 64): the other 32 channels
    must keep their contents."""
    x = cc.uniform((2, 64, 9, 9), 4, "so/x")
    w = cc.kaiming((64, 64, 3, 3), 4, "so/w")
    big = torch.full((2, 96, 9, 9), 7.0, dtype=torch.bfloat16, device="cuda").contiguous(memory_format=torch.channels_last)
    view = big[:, 16:80]
    ops.conv2d_into(to_dev(x, "bf16"), to_dev(w, "bf16"), view, None, None, 1, 1)
    want = run_oracle(x, w, None, None, 1, 1, 1, "", "bf16")
    assert cc.rel_err(view.float().cpu().numpy(), want) <= cc.TOL_16BIT
    assert (big[:, :16] == 7.0).all() and (big[:, 80:] == 7.0).all()


def test_host_memory_tensors_are_staged_through_the_gpu():
    """device_id = -1 views: the library copies in, computes on the GPU, copies out and waits."""
    x = cc.uniform((2, 64, 9, 9), 5, "host/x")
    w = cc.kaiming((32, 64, 3, 3), 5, "host/w")
    b = cc.normal((32,), 5, "host/b", 0.1)
    out = np.full((2, 32, 9, 9), np.nan, np.float32)
    mk = lambda a: ffi.View(a.ctypes.data, a.shape, [s // 4 for s in a.strides], ffi.DTYPE_FLOAT32, -1)
    ffi.conv2d_raw(mk(x), mk(w), mk(b), None, mk(out), padding=(1, 1), epilogue=ffi.EPILOGUE_BIAS_RELU)
    want = oracle.conv2d(x, w, b, None, 1, 1, 1, "relu")
    assert cc.rel_err(out, want) <= cc.TOL_TF32


def test_large_host_batches_are_pipelined_in_chunks_with_identical_results(monkeypatch):
    """Host tensors above a few MB are cut into image chunks whose copy-in, kernels and copy-out overlap;
    the result must be bit-identical to the single-shot staging and match the oracle."""
    n = 36
    x = cc.uniform((n, 64, 32, 32), 5, "hostc/x")
    w = cc.kaiming((64, 64, 3, 3), 5, "hostc/w")
    b = cc.normal((64,), 5, "hostc/b", 0.1)
    r = cc.normal((n, 64, 32, 32), 5, "hostc/r")
    mk = lambda a: ffi.View(a.ctypes.data, a.shape, [s // 4 for s in a.strides], ffi.DTYPE_FLOAT32, -1)
    outs = []
    for chunks in ("1", "8", "5"):
        monkeypatch.setenv("TRACEA_B200_HOST_CHUNKS", chunks)
        out = np.full((n, 64, 32, 32), np.nan, np.float32)
        ffi.conv2d_raw(mk(x), mk(w), mk(b), mk(r), mk(out), padding=(1, 1), epilogue=ffi.EPILOGUE_BIAS_RESIDUAL_RELU)
        outs.append(out)
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])
    want = oracle.conv2d_gemm(cc.channels_last(x), w, b, r, 1, 1, 1, "relu")
    assert cc.rel_err(outs[1], want) <= cc.TOL_TF32


def test_work_is_enqueued_on_the_callers_stream():
    x = to_dev(cc.uniform((4, 64, 14, 14), 6, "st/x"), "bf16")
    w = to_dev(cc.kaiming((64, 64, 3, 3), 6, "st/w"), "bf16")
    want = ops.conv2d_nchw(x, w, padding=1)
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        got = ops.conv2d_nchw(x, w, padding=1)
    s.synchronize()
    assert torch.equal(got, want)


def test_five_argument_entry_point_adds_bias_when_given():
    import ctypes
    x = cc.uniform((1, 64, 8, 8), 7, "v0/x")
    w = cc.kaiming((64, 64, 3, 3), 7, "v0/w")
    b = cc.normal((64,), 7, "v0/b", 0.3)
    tx, tw, tb = to_dev(x, "bf16"), to_dev(w, "bf16"), torch.from_numpy(b).cuda()
    out = torch.empty((1, 64, 8, 8), dtype=torch.bfloat16, device="cuda", memory_format=torch.channels_last)
    vo, vb = ops._view(out), ops._view(tb)
    p = ffi.Conv2dParamsV0(1, 1, 1, 1, 1, 1, 1, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    st = ffi.load().tracea_conv2d_v0(ops._view(tx).c, ops._view(tw).c, ctypes.byref(vb.c), ctypes.byref(vo.c), p)
    assert st == ffi.SUCCESS
    torch.cuda.synchronize()
    want = run_oracle(x, w, b, None, 1, 1, 1, "bias", "bf16")
    assert cc.rel_err(out.float().cpu().numpy(), want) <= cc.TOL_16BIT


def test_unsupported_on_device_configurations_report_a_status():
    x = to_dev(cc.uniform((1, 64, 40, 40), 8, "un/x"), "bf16")
    w = to_dev(cc.kaiming((64, 64, 3, 3), 8, "un/w"), "bf16")
    with pytest.raises(ffi.TraceaError) as e:
        ops.conv2d_nchw(x, w, stride=9)            # the TMA traversal stride tops out at 8
    assert e.value.status == ffi.UNSUPPORTED_CONFIG
    with pytest.raises(ffi.TraceaError) as e:
        ops.conv2d_nchw(x, w, groups=2)
    assert e.value.status == ffi.UNSUPPORTED_CONFIG


def test_large_m_many_waves():
    """M = 2^20 output pixels (8192 tiles, many persistent-loop iterations per CTA)."""
    x = cc.uniform((16, 64, 256, 256), 9, "big/x")
    w = cc.kaiming((64, 64, 1, 1), 9, "big/w")
    got = run_gpu(x, w, None, None, 1, 0, 1, "", "bf16")
    rng = np.random.default_rng(9)
    idx = np.stack([rng.integers(0, s, 20000) for s in got.shape], axis=1)
    want = oracle.conv2d_points(cc.round_to(x, "bf16"), cc.round_to(w, "bf16"), idx)
    vals = got[idx[:, 0], idx[:, 1], idx[:, 2], idx[:, 3]]
    assert np.abs(vals - want).max() <= cc.TOL_16BIT * np.abs(want).max()


# --------------------------------------------------------------------------- tiles split over K (opt-in schedule)
_SPLIT_K_SCRIPT = r"""
import sys
import numpy as np, torch
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + "/tests")
import convcases as cc
from oracle import oracle
from tracea_b200 import ffi, ops
cl = lambda t: t.contiguous(memory_format=torch.channels_last)
dev = lambda a: cl(torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16).cuda())
# N, C, H, K, R, pad, epilogue: more than one wave with a partial last wave (two pieces per split tile, CTA pairs and
# single CTAs), and fewer tiles than SMs (three and more pieces per tile, two-row-block tiles)
CASES = [(256, 256, 14, 256, 3, 1, "bias+relu"), (200, 1024, 14, 256, 1, 0, "bias+residual+relu"),
         (64, 512, 7, 512, 3, 1, "bias+relu"), (16, 2048, 7, 512, 1, 0, "bias+silu"), (40, 512, 14, 128, 3, 1, "relu"),
         (150, 256, 14, 1024, 1, 0, "bias+residual+relu"), (3, 64, 56, 64, 3, 1, "bias+relu"),
         (8, 256, 56, 64, 3, 1, "bias+residual+relu")]   # two-row-block tiles cut in two or three: both groups finish a tile
for N, C, H, K, R, pad, epi in CASES:
    x = np.abs(cc.normal((N, C, H, H), 3, "sk/x")); w = cc.kaiming((K, C, R, R), 3, "sk/w")
    b = cc.normal((K,), 3, "sk/b", 0.05); r = cc.normal((N, K, H, H), 3, "sk/r")
    ub, ur = "bias" in epi, "residual" in epi
    act = next((o for o in epi.split("+") if o in ("relu", "silu")), "none")
    outs = []
    for rep in range(2):   # twice: the second launch finds the counters the first one left behind
        got = ops.conv2d_nchw(dev(x), dev(w), torch.from_numpy(b).cuda() if ub else None, dev(r) if ur else None,
                              1, pad, 1, 1, epi)
        torch.cuda.synchronize()
        outs.append(got)
    assert torch.equal(outs[0], outs[1]), "not reproducible"
    want = oracle.conv2d_gemm(cc.channels_last(cc.round_to(x, "bf16")), cc.round_to(w, "bf16"), b if ub else None,
                              cc.channels_last(cc.round_to(r, "bf16")) if ur else None, 1, pad, 1, act)
    err = cc.rel_err(outs[0].float().cpu().numpy(), cc.round_to(np.ascontiguousarray(want), "bf16"))
    assert err <= cc.TOL_16BIT, (N, C, H, K, R, err)
assert ffi.load().tracea_b200_device_status(0) == 0
print("split-k ok")
"""


def test_tiles_split_over_k_match_the_oracle_and_repeat_bit_for_bit():
    """The K-split schedule is off by default (TRACEA_B200_SPLIT_K=1 turns it on, read once per process), so it is
    exercised in a child process: ResNet-sized layers whose last wave is partly filled or that have fewer tiles
    than SMs, against the oracle, each launched twice with identical bits (the pieces are summed in piece order
    whichever of them finishes last)."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, TRACEA_B200_SPLIT_K="1")
    res = subprocess.run([sys.executable, "-c", _SPLIT_K_SCRIPT, root], env=env, capture_output=True, text=True,
                         timeout=600)
    assert res.returncode == 0 and "split-k ok" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]


# --------------------------------------------------------------------------- resident-filter kernel (stride-1 small filters, C = 64)
RESIDENT = [
    # N, H, W, K, R, S, pad, dtype, epilogue
    (32, 56, 56, 64, 3, 3, 1, "bf16", "bias+relu"),      # the reference's benchmark layer at batch 32: full + short tiles
    (33, 56, 56, 64, 3, 3, 1, "bf16", "bias+relu"),      # odd tile counts: one CTA of the last pair has no tile
    (40, 56, 56, 40, 3, 3, 1, "f16", "bias+silu"),       # K_out < 64: zero filter rows, masked stores
    (64, 40, 31, 64, 3, 3, 1, "bf16", ""),               # odd width, no bias
    (64, 40, 31, 64, 3, 3, 0, "bf16", "bias"),           # no padding: the dummy columns are real input columns
    (64, 30, 50, 64, 2, 3, (1, 1), "bf16", "gelu"),      # 2x3 filter, one output row more than input rows
    (200, 28, 28, 64, 3, 3, 1, "bf16", "relu"),
    (150, 20, 120, 48, 3, 3, (0, 1), "f16", "bias+relu"),   # wide rows: three-block tiles, no short tile
]


@pytest.mark.parametrize("case", RESIDENT, ids=lambda c: "N%dH%dW%dK%dR%dS%d" % c[:6])
def test_resident_filter_kernel_matches_the_oracle(case):
    """Stride-1 small filters over 64-channel 16-bit activations take the kernel that keeps the filter bank in
    shared memory and reads every tap from one halo'd window (conv2d_window_sm100.cuh): full tensors against the
    oracle, and the launch counter shows that this kernel -- not the general one -- produced them."""
    N, H, W, K, R, S, pad, dtype, epi = case
    x = cc.normal((N, 64, H, W), 6, "rf/x")
    w = cc.kaiming((K, 64, R, S), 6, "rf/w")
    b = cc.normal((K,), 6, "rf/b", 0.1)
    before = ffi.launch_count_of(ffi.KERNEL_RESIDENT_FILTER)
    check(x, w, b, None, 1, pad, 1, epi, dtype)
    assert ffi.launch_count_of(ffi.KERNEL_RESIDENT_FILTER) == before + 1


def test_resident_filter_kernel_writes_strided_views_and_agrees_with_the_general_kernel():
    """Output as a channel slice of a wider buffer (pixel pitch 96): the gaps keep their contents; and the general
    kernel (smaller batch, same images) gives the same values up to the summation order inside an MMA."""
    n = 40
    x = cc.normal((n, 64, 56, 56), 7, "rf2/x")
    w = cc.kaiming((64, 64, 3, 3), 7, "rf2/w")
    b = cc.normal((64,), 7, "rf2/b", 0.1)
    tx, tw, tb = to_dev(x, "bf16"), to_dev(w, "bf16"), torch.from_numpy(b).cuda()
    big = torch.full((n, 96, 56, 56), 7.0, dtype=torch.bfloat16, device="cuda").contiguous(memory_format=torch.channels_last)
    view = big[:, 16:80]
    before = ffi.launch_count_of(ffi.KERNEL_RESIDENT_FILTER)
    ops.conv2d_into(tx, tw, view, tb, None, 1, 1, 1, 1, ffi.EPILOGUE_BIAS_RELU)
    torch.cuda.synchronize()
    assert ffi.launch_count_of(ffi.KERNEL_RESIDENT_FILTER) == before + 1
    assert (big[:, :16] == 7.0).all() and (big[:, 80:] == 7.0).all()
    general = ops.conv2d_nchw(tx[:2], tw, tb, None, 1, 1, 1, 1, "bias+relu")     # 2 images: too few tiles, general kernel
    assert ffi.launch_count_of(ffi.KERNEL_RESIDENT_FILTER) == before + 1
    a, g = view[:2].float(), general.float()
    assert float((a - g).abs().max()) <= 2.0 ** -7 * float(g.abs().max())
    want = run_oracle(x, w, b, None, 1, 1, 1, "bias+relu", "bf16")
    assert cc.rel_err(view.float().cpu().numpy(), want) <= cc.TOL_16BIT


# --------------------------------------------------------------------------- row-band kernel (few-channel images)
ROW_BAND = [
    # N, C, H, W, K, R, S, stride, pad, dil, dtype, epilogue
    (2, 3, 64, 230, 64, 7, 7, 2, 3, 1, "bf16", "bias+relu"),          # the RGB stem shape family: 4-channel pixels, stride 2
    (3, 3, 224, 224, 64, 7, 7, 2, 3, 1, "f16", "bias+relu"),          # ResNet-50 conv1 itself
    (2, 4, 20, 250, 16, 2, 8, (1, 2), (0, 3), 1, "bf16", ""),         # 8-wide filter row: both K slices full; K_out 16
    (1, 8, 30, 120, 40, 3, 3, 1, 1, 1, "bf16", "bias+silu"),          # 8-channel pixels, stride 1; K_out 40: clipped stores
    (1, 6, 18, 100, 64, 5, 5, 1, 2, 1, "f16", "gelu"),                # 6 channels padded to 8: three K slices per filter row
    (1, 3, 20, 520, 32, 3, 3, 2, 1, 1, "bf16", "bias"),               # Wo = 260: three column tiles, the last one ragged
    (1, 3, 40, 240, 24, 3, 5, (3, 2), (2, 2), (2, 1), "bf16", "relu"),   # vertical stride 3, vertical dilation 2
    (5, 1, 33, 200, 8, 4, 6, (1, 2), (3, 2), 1, "bf16", "bias+relu"),    # one channel; more padding than the filter needs
    (1, 3, 9, 224, 64, 7, 7, 2, 3, 1, "bf16", "bias+relu"),           # fewer output rows than a band holds
]


@pytest.mark.parametrize("case", ROW_BAND, ids=lambda c: "N%dC%dH%dW%dK%dR%dS%d" % c[:7])
@pytest.mark.parametrize("channels_last", [True, False])
def test_row_band_kernel_matches_the_oracle(case, channels_last):
    """16-bit images of up to 8 channels whose horizontal step is 16 bytes of channel-padded input take the kernel
    that keeps bands of input rows in shared memory and reads the im2col matrix through overlapping-row descriptors
    (conv2d_rowband_sm100.cuh): full tensors against the oracle, from channels-last and from NCHW memory, and the
    launch counter shows which kernel produced them."""
    N, C, H, W, K, R, S, stride, pad, dil, dtype, epi = case
    x = cc.normal((N, C, H, W), 8, "rb/x")
    w = cc.kaiming((K, C, R, S), 8, "rb/w")
    b = cc.normal((K,), 8, "rb/b", 0.1)
    before = ffi.launch_count_of(ffi.KERNEL_ROW_BAND)
    check(x, w, b, None, stride, pad, dil, epi, dtype, channels_last=channels_last, out_channels_last=True)
    assert ffi.launch_count_of(ffi.KERNEL_ROW_BAND) == before + 1


def test_row_band_kernel_agrees_with_the_general_kernel_on_a_zero_padded_image():
    """The same RGB image stored with 8 channels (5 of them zero) does not qualify (stride 2 over 16-byte pixels) and
    takes the general kernel: same values up to the summation order inside an MMA."""
    n = 4
    x = cc.normal((n, 3, 96, 224), 9, "rb2/x")
    w = cc.kaiming((64, 3, 7, 7), 9, "rb2/w")
    b = cc.normal((64,), 9, "rb2/b", 0.1)
    x8 = np.zeros((n, 8, 96, 224), np.float32)
    x8[:, :3] = x
    w8 = np.zeros((64, 8, 7, 7), np.float32)
    w8[:, :3] = w
    tb = torch.from_numpy(b).cuda()
    before = ffi.launch_count_of(ffi.KERNEL_ROW_BAND)
    band = ops.conv2d_nchw(to_dev(x, "bf16"), to_dev(w, "bf16"), tb, None, 2, 3, 1, 1, "bias+relu")
    assert ffi.launch_count_of(ffi.KERNEL_ROW_BAND) == before + 1
    general = ops.conv2d_nchw(to_dev(x8, "bf16"), to_dev(w8, "bf16"), tb, None, 2, 3, 1, 1, "bias+relu")
    assert ffi.launch_count_of(ffi.KERNEL_ROW_BAND) == before + 1
    torch.cuda.synchronize()
    a, g = band.float(), general.float()
    assert float((a - g).abs().max()) <= 2.0 ** -7 * float(g.abs().max())


def test_row_band_kernel_random_cases():
    """Seeded random few-channel layers around the row-band kernel's conditions (channels, filter widths up to four
    K slices, vertical stride / dilation, paddings larger and smaller than the filter needs, ragged column tiles,
    K_out below 64, both memory layouts): parity with the oracle, and most of them must have taken that kernel."""
    rng = np.random.default_rng(77)
    took = 0
    total = 40
    for i in range(total):
        C = int(rng.integers(1, 9))
        sw = 2 if C <= 4 else 1
        S = int(rng.integers(2, 9 if C > 4 else 13))
        R = int(rng.integers(1, 8))
        sh, dh = int(rng.integers(1, 4)), int(rng.integers(1, 3))
        W = int(rng.integers(80, 420)) * (2 if sw == 2 else 1)
        H = int(rng.integers((R - 1) * dh + 1, (R - 1) * dh + 40))
        K = int(rng.integers(1, 9)) * 8
        ph, pw = int(rng.integers(0, R + 1)), int(rng.integers(0, S + 2))
        N = int(rng.integers(1, 4))
        dtype = str(rng.choice(["bf16", "f16"]))
        epi = str(rng.choice(["", "bias", "bias+relu", "silu", "bias+gelu".replace("bias+gelu", "gelu")]))
        cl = bool(rng.integers(0, 2))
        if (W + 2 * pw - S) // sw + 1 < 1 or (H + 2 * ph - dh * (R - 1) - 1) // sh + 1 < 1:
            continue
        x = cc.normal((N, C, H, W), 100 + i, "rbf/x")
        w = cc.kaiming((K, C, R, S), 100 + i, "rbf/w")
        b = cc.normal((K,), 100 + i, "rbf/b", 0.1)
        before = ffi.launch_count_of(ffi.KERNEL_ROW_BAND)
        check(x, w, b, None, (sh, sw), (ph, pw), (dh, 1), epi, dtype, channels_last=cl, out_channels_last=True)
        took += ffi.launch_count_of(ffi.KERNEL_ROW_BAND) - before
    assert took >= total // 2, took

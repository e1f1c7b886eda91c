"""ConvTranspose2d, GEMM and weight prepacking on a B200, against the CPU oracle, through the C ABI.

Tolerances are those of the conv path: max|out - ref| <= 1e-2 * max|ref| for fp16 / bf16 inputs with fp32
accumulation, 5e-3 * max|ref| for fp32 inputs computed as TF32. The oracle gets the inputs already rounded to the
storage type and its result is rounded once at the end.
"""
import os

import numpy as np
import pytest
import torch

import convcases as cc
from golden.make_golden_next_ops import CONVT_CASES, GEMM_CASES
from oracle import oracle
from tracea_b200 import ffi, ops

pytestmark = pytest.mark.gpu

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "next_ops_golden.npz"))
TORCH_DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
# launch-count assertions describe the default configuration; bring-up knobs may force extra staging kernels
DEFAULT_CONFIG = not any(k.startswith("TRACEA_B200_") for k in os.environ)


def dev(a, dtype):
    return torch.from_numpy(np.ascontiguousarray(a)).to(TORCH_DT[dtype]).cuda()


def host(t):
    torch.cuda.synchronize()
    assert ffi.load().tracea_b200_device_status(0) == 0
    return t.float().cpu().numpy()


def split_epi(epi):
    ops_ = [o for o in (epi or "").split("+") if o]
    act = next((o for o in ops_ if o in ("relu", "silu", "gelu")), "none")
    return "bias" in ops_, "residual" in ops_, act


# --------------------------------------------------------------------------- ConvTranspose2d
def convt_both(x, w, b, res, stride, padding, opad, epi, dtype):
    use_b, use_r, act = split_epi(epi)
    got = host(ops.conv_transpose2d(dev(x, dtype), dev(w, dtype), torch.from_numpy(b).cuda() if use_b else None,
                                    dev(res, dtype) if use_r else None, epi or None, stride, padding, opad))
    want = oracle.conv_transpose2d(cc.round_to(x, dtype), cc.round_to(w, dtype), b if use_b else None,
                                   cc.round_to(res, dtype) if use_r else None, stride, padding, opad, act)
    return got, cc.round_to(want, dtype)


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("name", sorted(CONVT_CASES))
def test_conv_transpose_golden_fixtures(name, dtype):
    spec = CONVT_CASES[name]
    g = {k: GOLDEN["convt/%s/%s" % (name, k)] for k in ("x", "w", "b", "res", "out")}
    got, want = convt_both(g["x"], g["w"], g["b"], g["res"], spec[7], spec[8], spec[9], spec[10], dtype)
    assert got.shape == want.shape == g["out"].shape
    assert cc.rel_err(got, want) <= cc.tol_for(dtype)
    # and against the committed torch output itself (inputs not pre-rounded: one more rounding of slack)
    assert cc.rel_err(got, g["out"]) <= 2.5 * cc.tol_for(dtype)


# decoder-style upsampling layers (the shapes of the reference's VAE-decoder presets, src/optimizer/benchmark.rs:568-583,
# at reduced batch / resolution) and shapes that exercise several M tiles and wide channel counts
@pytest.mark.parametrize("case", [
    (2, 16, 16, 128, 64, 4, 4, (2, 2), (1, 1), (0, 0), "bias+relu"),
    (1, 32, 32, 64, 32, 3, 3, (2, 2), (1, 1), (1, 1), "bias+silu"),
    (4, 14, 14, 256, 256, 2, 2, (2, 2), (0, 0), (0, 0), "bias+residual+relu"),
    (2, 9, 11, 32, 24, 5, 3, (3, 2), (2, 1), (2, 1), "bias"),
    (1, 20, 20, 64, 128, 3, 3, (1, 1), (1, 1), (0, 0), "relu"),
])
def test_conv_transpose_larger_shapes_bf16(case):
    N, H, W, C, K, R, S, stride, padding, opad, epi = case
    x = cc.normal((N, H, W, C), 3, "ct/x")
    w = cc.normal((K, R, S, C), 3, "ct/w", (1.0 / (C * R * S)) ** 0.5)
    b = cc.normal((K,), 3, "ct/b", 0.1)
    shape = oracle.conv_transpose_out_shape(x.shape, w.shape, stride, padding, opad)
    res = cc.normal(shape, 3, "ct/res")
    got, want = convt_both(x, w, b, res, stride, padding, opad, epi, "bf16")
    assert cc.rel_err(got, want) <= cc.TOL_16BIT


def test_conv_transpose_reads_the_reference_kernels_crsk_weight_memory():
    name = "s2_p1_4x4_decoder"
    spec = CONVT_CASES[name]
    g = {k: GOLDEN["convt/%s/%s" % (name, k)] for k in ("x", "w")}
    w = dev(g["w"], "bf16")
    crsk = w.permute(3, 1, 2, 0).contiguous()            # memory [C][R][S][K], what the reference's kernel indexes
    a = ops.conv_transpose2d(dev(g["x"], "bf16"), w, stride=spec[7], padding=spec[8], output_padding=spec[9])
    b = ops.conv_transpose2d(dev(g["x"], "bf16"), crsk.permute(3, 1, 2, 0), stride=spec[7], padding=spec[8],
                             output_padding=spec[9])
    assert torch.equal(a, b)


@pytest.mark.parametrize("C", [32, 64, 192])    # 64-byte k-chunks: phase filters are gathered; 128-byte: read in place
def test_conv_transpose_stride1_is_the_conv_with_flipped_taps_bit_exactly(C):
    x = cc.normal((2, 10, 10, C), 5, "ctf/x")
    w = cc.normal((16, 3, 3, C), 5, "ctf/w", 0.06)
    tx, tw = dev(x, "bf16"), dev(w, "bf16")
    a = ops.conv_transpose2d(tx, tw, stride=1, padding=1)
    b = ops.conv2d(tx, torch.flip(tw, (1, 2)).contiguous(), stride=1, padding=1)   # pad' = R - 1 - pad = 1
    assert torch.equal(a, b)


def test_conv_transpose_host_tensors_and_strided_output():
    name = "s2_p1_3x3_opad"
    spec = CONVT_CASES[name]
    g = {k: GOLDEN["convt/%s/%s" % (name, k)] for k in ("x", "w", "b", "out")}
    x, w, b = torch.from_numpy(g["x"]), torch.from_numpy(g["w"]), torch.from_numpy(g["b"])
    got = ops.conv_transpose2d(x, w, b, None, "bias", spec[7], spec[8], spec[9])      # CPU tensors: staged by the library
    assert not got.is_cuda
    assert cc.rel_err(got.numpy(), g["out"]) <= cc.TOL_TF32
    # device output with gaps between pixels: the gaps keep their contents
    big = torch.full((2, 10, 12, 32), 7.0, device="cuda")
    view = big[..., :16]
    dx, dw, db = x.cuda(), w.cuda(), b.cuda()
    ffi.conv_transpose2d_raw(ops._view(dx), ops._view(dw), ops._view(db), None, ops._view(view),
                             spec[7], spec[8], spec[9], epilogue=ffi.EPILOGUE_BIAS_ADD,
                             stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert cc.rel_err(view.cpu().numpy(), g["out"]) <= cc.TOL_TF32
    assert bool((big[..., 16:] == 7.0).all())


# --------------------------------------------------------------------------- GEMM
def gemm_want(a, bm, b, res, epi, dtype):
    use_b, use_r, act = split_epi(epi)
    want = oracle.gemm(cc.round_to(a, dtype), cc.round_to(bm, dtype), b if use_b else None,
                       cc.round_to(res, dtype) if use_r else None, act)
    return cc.round_to(want, dtype)


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("name", sorted(GEMM_CASES))
def test_gemm_golden_fixtures(name, dtype):
    g = {k: GOLDEN["gemm/%s/%s" % (name, k)] for k in ("a", "bm", "b", "res", "out")}
    epi = GEMM_CASES[name][3]
    use_b, use_r, _ = split_epi(epi)
    got = host(ops.gemm(dev(g["a"], dtype), dev(g["bm"], dtype), torch.from_numpy(g["b"]).cuda() if use_b else None,
                        epi or None, dev(g["res"], dtype) if use_r else None))
    assert cc.rel_err(got, gemm_want(g["a"], g["bm"], g["b"], g["res"], epi, dtype)) <= cc.tol_for(dtype)
    assert cc.rel_err(got, g["out"]) <= 2.5 * cc.tol_for(dtype)


@pytest.mark.parametrize("layout", ["row_major_b", "transposed_b", "prepacked_b", "column_major_a", "column_major_c"])
def test_gemm_operand_layouts_give_identical_results(layout):
    M, K, N = 1000, 512, 384
    a = cc.normal((M, K), 7, "g/a")
    bm = cc.normal((K, N), 7, "g/b", K ** -0.5)
    bias = cc.normal((N,), 7, "g/bias", 0.1)
    ta, tb, tbias = dev(a, "bf16"), dev(bm, "bf16"), torch.from_numpy(bias).cuda()
    base = ops.gemm(ta, tb, tbias, "bias+relu")
    assert cc.rel_err(host(base), gemm_want(a, bm, bias, None, "bias+relu", "bf16")) <= cc.TOL_16BIT
    if layout == "transposed_b":
        other = ops.gemm(ta, tb.t().contiguous().t(), tbias, "bias+relu")
    elif layout == "prepacked_b":
        packed = ops.prepack_gemm_b(tb)
        assert packed.stride() == (1, K) and torch.equal(packed, tb)
        other = ops.gemm(ta, packed, tbias, "bias+relu")
    elif layout == "column_major_a":
        other = ops.gemm(ta.t().contiguous().t(), tb, tbias, "bias+relu")
    elif layout == "column_major_c":
        out = torch.empty((N, M), dtype=torch.bfloat16, device="cuda").t()
        ffi.gemm_raw(ops._view(ta), ops._view(tb), ops._view(tbias), None, ops._view(out), ffi.EPILOGUE_BIAS_RELU,
                     torch.cuda.current_stream().cuda_stream)
        other = out
    else:
        other = ops.gemm(ta, tb, tbias, "bias+relu")
    assert torch.equal(other, base)


@pytest.mark.parametrize("shape", [(700, 256, 4096), (300, 128, 2560 + 64), (129, 64, 9 * 256 + 8)])
def test_gemm_wide_outputs_walk_the_tiles_in_panels(shape):
    """More than 8 column tiles: the kernel walks panels of 8 (the last one narrower); every tile is still visited once."""
    M, K, N = shape
    a = cc.normal((M, K), 12, "gw/a")
    bm = cc.normal((K, N), 12, "gw/b", K ** -0.5)
    bias = cc.normal((N,), 12, "gw/bias", 0.1)
    got = host(ops.gemm(dev(a, "bf16"), dev(bm, "bf16"), torch.from_numpy(bias).cuda(), "bias"))
    assert cc.rel_err(got, gemm_want(a, bm, bias, None, "bias", "bf16")) <= cc.TOL_16BIT


def test_gemm_reads_a_padded_pitch_b_in_place():
    M, K, N = 300, 128, 72
    a = dev(cc.normal((M, K), 8, "gp/a"), "bf16")
    storage = torch.zeros((N, K + 64), dtype=torch.bfloat16, device="cuda")       # [N][K] rows with a 64-element gap
    storage[:, :K] = dev(cc.normal((N, K), 8, "gp/b", K ** -0.5), "bf16")
    b = storage[:, :K].t()                                                          # (K, N), strides (1, K + 64)
    before = ffi.load().tracea_b200_launch_count()
    got = ops.gemm(a, b)
    if DEFAULT_CONFIG:
        assert ffi.load().tracea_b200_launch_count() - before == 1                  # no transpose kernel ran
    assert torch.equal(got, ops.gemm(a, b.contiguous()))


def test_gemm_fc_head_shape_and_host_tensors():
    """The ResNet-50 classifier head as a GEMM: [N, 2048] x [2048, 1000] + bias."""
    a = np.abs(cc.normal((64, 2048), 9, "fc/a"))
    bm = cc.normal((2048, 1000), 9, "fc/b", 2048 ** -0.5)
    bias = cc.normal((1000,), 9, "fc/bias", 0.05)
    got = host(ops.gemm(dev(a, "bf16"), dev(bm, "bf16"), torch.from_numpy(bias).cuda(), "bias"))
    assert cc.rel_err(got, gemm_want(a, bm, bias, None, "bias", "bf16")) <= cc.TOL_16BIT
    cpu = ops.gemm(torch.from_numpy(a[:8]), torch.from_numpy(bm), torch.from_numpy(bias), "bias")   # staged by the library
    assert not cpu.is_cuda
    assert cc.rel_err(cpu.numpy(), gemm_want(a[:8], bm, bias, None, "bias", "f32")) <= cc.TOL_TF32


# --------------------------------------------------------------------------- prepacking
@pytest.mark.parametrize("shape", [(64, 32, 3, 3), (24, 16, 1, 1), (16, 3, 7, 7)])
def test_prepacked_conv_weights_are_read_in_place_with_identical_results(shape):
    K, C, R, S = shape
    w = dev(cc.normal(shape, 11, "pp/w", (C * R * S) ** -0.5), "bf16")          # OIHW-contiguous
    packed = ops.prepack_conv2d_weight(w)
    Cp = (C + 7) // 8 * 8
    assert tuple(packed.shape) == (K, Cp, R, S) and packed.stride() == (R * S * Cp, 1, S * Cp, Cp)
    assert torch.equal(packed[:, :C], w) and bool((packed[:, C:] == 0).all())
    x = dev(cc.normal((2, C, 12, 12), 11, "pp/x"), "bf16").contiguous(memory_format=torch.channels_last)
    if Cp != C:       # the activations carry the padded channels too
        xp = torch.zeros((2, Cp, 12, 12), dtype=x.dtype, device="cuda").contiguous(memory_format=torch.channels_last)
        xp[:, :C] = x
    else:
        xp = x
    a = ops.conv2d_nchw(x, w, None, None, 1, R // 2)
    b = ops.conv2d_nchw(xp, packed, None, None, 1, R // 2)
    assert torch.equal(a, b)


# --------------------------------------------------------------------------- torch.nn front end
@pytest.mark.parametrize("cfg", [dict(cin=64, cout=96, k=3, stride=1, padding=1, bias=True),
                                 dict(cin=3, cout=32, k=7, stride=2, padding=3, bias=False),
                                 dict(cin=32, cout=64, k=3, stride=1, padding=2, dilation=2, bias=True)])
def test_nn_module_is_a_drop_in_for_conv2d(cfg):
    from tracea_b200 import nn as tnn
    torch.manual_seed(3)
    m = tnn.TraceaConv2d(cfg["cin"], cfg["cout"], cfg["k"], stride=cfg["stride"], padding=cfg["padding"],
                         dilation=cfg.get("dilation", 1), bias=cfg["bias"]).cuda().to(torch.bfloat16)
    x = torch.randn(2, cfg["cin"], 20, 20, device="cuda", dtype=torch.bfloat16)
    before = ffi.load().tracea_b200_launch_count()
    y1 = m(x)
    first = ffi.load().tracea_b200_launch_count() - before
    y2 = m(x.contiguous(memory_format=torch.channels_last))
    second = ffi.load().tracea_b200_launch_count() - before - first
    assert torch.equal(y1, y2.contiguous())
    if cfg["cin"] % 8 == 0 and DEFAULT_CONFIG:
        assert second == 1                       # packed weights cached, channels-last input: the conv kernel only
    want = oracle.conv2d(x.float().cpu().numpy(), m.weight.detach().float().cpu().numpy(),
                         m.bias.detach().float().cpu().numpy() if cfg["bias"] else None, None, cfg["stride"],
                         cfg["padding"], cfg.get("dilation", 1), "none")
    assert cc.rel_err(host(y1), cc.round_to(want, "bf16")) <= cc.TOL_16BIT
    with pytest.raises(NotImplementedError):
        tnn.TraceaConv2d(8, 8, 3, groups=2).cuda()(torch.randn(1, 8, 5, 5, device="cuda"))


def test_conv_transpose_phases_overlap_and_replay_from_a_cuda_graph():
    """The phase launches of a transposed convolution do not depend on each other and are issued as a chain of
    programmatic launches that may run side by side (the first waits before it lets the next one start, the later
    ones wait at their end). Many waves per phase, a residual, back-to-back calls into the same output, and the same
    call captured into a CUDA graph and replayed: always the bits of a run with the overlap switched off."""
    import subprocess
    import sys
    rng = np.random.default_rng(5)
    x = torch.from_numpy(rng.standard_normal((48, 32, 32, 128)).astype(np.float32)).to(torch.bfloat16).cuda()
    w = torch.from_numpy((rng.standard_normal((128, 4, 4, 128)) * 0.02).astype(np.float32)).to(torch.bfloat16).cuda()
    b = torch.from_numpy(rng.standard_normal(128).astype(np.float32) * 0.1).cuda()
    r = torch.from_numpy(rng.standard_normal((48, 64, 64, 128)).astype(np.float32)).to(torch.bfloat16).cuda()
    run = lambda: ops.conv_transpose2d(x, w, b, r, "bias+residual+relu", stride=2, padding=1)
    first = run()
    for _ in range(5):
        again = run()
    torch.cuda.synchronize()
    assert torch.equal(first, again)
    f32 = lambda t: t.float().cpu().numpy()
    want = oracle.conv_transpose2d(f32(x[:3]), f32(w), b.cpu().numpy(), f32(r[:3]), 2, 1, 0, "relu")   # three images
    assert cc.rel_err(f32(first[:3]), cc.round_to(np.ascontiguousarray(want), "bf16")) <= cc.TOL_16BIT
    # captured and replayed
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        run()                                  # warm on the capture stream
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            captured = run()
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        captured.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(captured, first)
    # the same call with the overlap switched off, in a child process (the switch is read once per process)
    script = (
        "import sys, numpy as np, torch\n"
        "sys.path.insert(0, sys.argv[1])\n"
        "from tracea_b200 import ops\n"
        "rng = np.random.default_rng(5)\n"
        "x = torch.from_numpy(rng.standard_normal((48, 32, 32, 128)).astype(np.float32)).to(torch.bfloat16).cuda()\n"
        "w = torch.from_numpy((rng.standard_normal((128, 4, 4, 128)) * 0.02).astype(np.float32)).to(torch.bfloat16).cuda()\n"
        "b = torch.from_numpy(rng.standard_normal(128).astype(np.float32) * 0.1).cuda()\n"
        "r = torch.from_numpy(rng.standard_normal((48, 64, 64, 128)).astype(np.float32)).to(torch.bfloat16).cuda()\n"
        "o = ops.conv_transpose2d(x, w, b, r, 'bias+residual+relu', stride=2, padding=1)\n"
        "torch.cuda.synchronize()\n"
        "np.save(sys.argv[2], o.view(torch.int16).cpu().numpy())\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = os.path.join(os.environ.get("TMPDIR", "/tmp"), "tb200_ct_serial_%d.npy" % os.getpid())
    res = subprocess.run([sys.executable, "-c", script, root, path], env=dict(os.environ, TRACEA_B200_PDL="0"),
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    serial = np.load(path)
    os.remove(path)
    assert np.array_equal(serial, first.view(torch.int16).cpu().numpy())

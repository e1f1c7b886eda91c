"""Writes tests/golden/conv2d_golden.npz: small known-answer cases for the Conv2d path.

The reference's own tests hold no golden vectors for conv (examples/verify_conv2d.rs and
examples/jit_conv_verify.py draw unseeded random inputs and only print / threshold the error).
Its comparison target, and what its Python operator returns at run time, is
torch.nn.functional.conv2d (examples/jit_conv_verify.py:20-26, tracea-python/src/conv2d.rs:80-136),
so the fixtures are that function's fp32 CPU output on seeded inputs, with the fused epilogue
(bias -> residual -> activation; formulas of src/kernels/gpu/epilogue.cuh:12-63) applied by torch ops.
The shapes of the reference's two conv checks are included under their own names.

Run from the repo root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import convcases as cc  # noqa: E402

# name: (N, C, H, W, K, R, S, stride, padding, dilation, epilogue, input distribution)
CASES = {
    "verify_conv2d_rs": (1, 32, 8, 8, 32, 3, 3, (1, 1), (1, 1), (1, 1), "", "uniform"),
    "jit_conv_verify_reduced": (2, 64, 7, 7, 64, 3, 3, (1, 1), (1, 1), (1, 1), "", "randn005"),
    "bias_relu_3x3": (2, 16, 10, 9, 24, 3, 3, (1, 1), (1, 1), (1, 1), "bias+relu", "uniform"),
    "strided_bias_silu": (2, 16, 12, 12, 24, 3, 3, (2, 2), (1, 1), (1, 1), "bias+silu", "normal"),
    "pointwise_bias_residual_relu": (2, 32, 6, 6, 40, 1, 1, (1, 1), (0, 0), (1, 1), "bias+residual+relu", "absnormal"),
    "stem_7x7_s2_c3": (1, 3, 20, 20, 8, 7, 7, (2, 2), (3, 3), (1, 1), "bias+relu", "normal"),
    "dilated_asym": (1, 8, 11, 13, 5, 3, 2, (2, 1), (2, 0), (2, 3), "gelu", "uniform"),
    "residual_only": (1, 8, 5, 5, 8, 3, 3, (1, 1), (1, 1), (1, 1), "residual", "uniform"),
    "pointwise_s2": (2, 16, 8, 8, 32, 1, 1, (2, 2), (0, 0), (1, 1), "bias", "normal"),
    "no_pad_3x3": (1, 8, 9, 9, 16, 3, 3, (1, 1), (0, 0), (1, 1), "silu", "uniform"),
}


def make_inputs(name, spec, seed=0):
    N, C, H, W, K, R, S, _, _, _, epi, dist = spec
    if dist == "uniform":
        x = cc.uniform((N, C, H, W), seed, name + "/x")
    elif dist == "randn005":
        x = cc.normal((N, C, H, W), seed, name + "/x", 0.05)
    elif dist == "absnormal":
        x = np.abs(cc.normal((N, C, H, W), seed, name + "/x"))
    else:
        x = cc.normal((N, C, H, W), seed, name + "/x")
    w = cc.kaiming((K, C, R, S), seed, name + "/w") if dist != "uniform" else cc.uniform((K, C, R, S), seed, name + "/w")
    b = cc.normal((K,), seed, name + "/b", 0.1)
    return x, w, b


def reference(x, w, b, res, spec):
    _, _, _, _, _, _, _, stride, padding, dilation, epi, _ = spec
    ops = [o for o in epi.split("+") if o]
    y = F.conv2d(torch.from_numpy(x), torch.from_numpy(w), None, stride, padding, dilation)
    if "bias" in ops:
        y = y + torch.from_numpy(b).view(1, -1, 1, 1)
    if "residual" in ops:
        y = y + torch.from_numpy(res)
    if "relu" in ops:
        y = torch.relu(y)
    if "silu" in ops:
        y = F.silu(y)
    if "gelu" in ops:
        y = F.gelu(y, approximate="tanh")
    return y.numpy()


def config1_digest():
    """Digest of benchmark config 1 at full size (fp32 NCHW x[1,64,56,56], OIHW w[64,64,3,3], stride 1,
    pad 1, bias, ReLU): every 7th output value, per-channel sums, and input checksums that let a test
    notice if the seeded generators ever drift."""
    x = cc.uniform((1, 64, 56, 56), 0, "cfg1/x")
    w = cc.uniform((64, 64, 3, 3), 0, "cfg1/w")
    b = cc.normal((64,), 0, "cfg1/b", 0.1)
    y = torch.relu(F.conv2d(torch.from_numpy(x), torch.from_numpy(w), torch.from_numpy(b), 1, 1)).numpy()
    return {
        "input_checksums": np.array([x.astype(np.float64).sum(), w.astype(np.float64).sum(),
                                     b.astype(np.float64).sum()]),
        "out_every7": y.reshape(-1)[::7].copy(),
        "out_channel_sums": y.astype(np.float64).sum(axis=(0, 2, 3)),
        "out_absmax": np.array([np.abs(y).max()]),
    }


def main():
    torch.set_num_threads(1)
    np.savez_compressed(os.path.join(HERE, "conv2d_cfg1_digest.npz"), **config1_digest())
    out = {}
    for name, spec in CASES.items():
        x, w, b = make_inputs(name, spec)
        y0 = F.conv2d(torch.from_numpy(x), torch.from_numpy(w), None, spec[7], spec[8], spec[9])
        res = cc.normal(tuple(y0.shape), 0, name + "/res")
        y = reference(x, w, b, res, spec)
        out[name + "/x"], out[name + "/w"], out[name + "/b"], out[name + "/res"], out[name + "/out"] = x, w, b, res, y
    np.savez_compressed(os.path.join(HERE, "conv2d_golden.npz"), **out)
    print("wrote", len(CASES), "cases,", os.path.getsize(os.path.join(HERE, "conv2d_golden.npz")), "bytes")


if __name__ == "__main__":
    main()

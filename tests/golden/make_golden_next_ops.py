"""Writes tests/golden/next_ops_golden.npz: small known-answer cases for ConvTranspose2d and GEMM.

The reference's own checks of these operators draw unseeded random inputs (examples/verify_conv_transpose.rs:78-97,
tests/numerical_parity.rs) and hold no golden vectors, so the fixtures are the fp32 CPU outputs of
torch.nn.functional.conv_transpose2d and torch.matmul -- the functions the reference's Python benchmarks compare
against (tracea-python/python/tracea/local_bench.py, examples/benchmark_compare.py) -- on seeded inputs, with the
fused epilogue (bias -> residual -> activation; src/kernels/gpu/epilogue.cuh:12-63) applied by torch ops.
Layouts are the reference's: x (N, H, W, C), w (K, R, S, C), out (N, Ho, Wo, K); a (M, K), b (K, N).

Run from the repo root:  python tests/golden/make_golden_next_ops.py
"""
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import convcases as cc  # noqa: E402

# name: (N, H, W, C, K, R, S, stride, padding, output_padding, epilogue)
CONVT_CASES = {
    "verify_conv_transpose_rs": (1, 2, 2, 1, 1, 2, 2, (1, 1), (0, 0), (0, 0), ""),
    "s1_p1_3x3": (2, 6, 5, 8, 16, 3, 3, (1, 1), (1, 1), (0, 0), "bias+relu"),
    "s2_p1_3x3_opad": (2, 5, 6, 8, 16, 3, 3, (2, 2), (1, 1), (1, 1), "bias"),
    "s2_p1_4x4_decoder": (1, 8, 8, 16, 8, 4, 4, (2, 2), (1, 1), (0, 0), "bias+silu"),
    "s2_2x2_upsample": (2, 4, 4, 8, 8, 2, 2, (2, 2), (0, 0), (0, 0), "residual+relu"),
    "s3_2x2_gaps": (1, 5, 5, 8, 8, 2, 2, (3, 3), (0, 0), (1, 1), "bias"),
    "asym_stride": (1, 6, 5, 8, 8, 3, 2, (2, 1), (1, 0), (1, 0), "gelu"),
    "crop_p3_5x5": (1, 6, 6, 8, 8, 5, 5, (1, 1), (3, 3), (0, 0), ""),
    "odd_channels": (1, 4, 4, 3, 5, 3, 3, (2, 2), (1, 1), (0, 0), "bias+residual+relu"),
}

# name: (M, K, N, epilogue)
GEMM_CASES = {
    "numerical_parity_small": (64, 64, 64, ""),
    "bias_relu": (70, 48, 40, "bias+relu"),
    "ragged": (33, 20, 9, "bias+residual"),
    "row_vector": (1, 64, 24, "silu"),
}


def epilogue(y, b, res, epi, channel_dim):
    ops = [o for o in epi.split("+") if o]
    if "bias" in ops:
        shape = [1] * y.ndim
        shape[channel_dim] = -1
        y = y + torch.from_numpy(b).view(*shape)
    if "residual" in ops:
        y = y + torch.from_numpy(res)
    if "relu" in ops:
        y = torch.relu(y)
    if "silu" in ops:
        y = F.silu(y)
    if "gelu" in ops:
        y = F.gelu(y, approximate="tanh")
    return y


def convt_inputs(name, spec, seed=0):
    N, H, W, C, K, R, S = spec[:7]
    x = cc.normal((N, H, W, C), seed, name + "/x")
    w = cc.normal((K, R, S, C), seed, name + "/w", (1.0 / (C * R * S)) ** 0.5)
    b = cc.normal((K,), seed, name + "/b", 0.1)
    return x, w, b


def main():
    torch.set_num_threads(1)
    out = {}
    for name, spec in CONVT_CASES.items():
        x, w, b = convt_inputs(name, spec)
        stride, padding, opad, epi = spec[7:]
        # torch wants x (N, C, H, W) and w (C_in, K_out, R, S)
        y0 = F.conv_transpose2d(torch.from_numpy(x).permute(0, 3, 1, 2), torch.from_numpy(w).permute(3, 0, 1, 2),
                                None, stride, padding, opad).permute(0, 2, 3, 1).contiguous()
        res = cc.normal(tuple(y0.shape), seed=0, tag=name + "/res")
        y = epilogue(y0, b, res, epi, 3).numpy()
        for k, v in (("x", x), ("w", w), ("b", b), ("res", res), ("out", y)):
            out["convt/%s/%s" % (name, k)] = v
    for name, (M, K, N, epi) in GEMM_CASES.items():
        a = cc.normal((M, K), 0, name + "/a")
        bm = cc.normal((K, N), 0, name + "/bm", (1.0 / K) ** 0.5)
        b = cc.normal((N,), 0, name + "/b", 0.1)
        res = cc.normal((M, N), 0, name + "/res")
        y = epilogue(torch.from_numpy(a) @ torch.from_numpy(bm), b, res, epi, 1).numpy()
        for k, v in (("a", a), ("bm", bm), ("b", b), ("res", res), ("out", y)):
            out["gemm/%s/%s" % (name, k)] = v
    path = os.path.join(HERE, "next_ops_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", len(CONVT_CASES), "+", len(GEMM_CASES), "cases,", os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()

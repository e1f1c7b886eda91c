"""Seeded random parity sweep: conv2d, conv_transpose2d and gemm over shapes, strides, paddings, dilations, dtypes,
memory layouts and every epilogue kind, each case against the CPU oracle through the C ABI.

Tolerances as everywhere: 1e-2 * max|ref| (fp16 / bf16), 5e-3 * max|ref| (fp32 computed as TF32). fp32 outputs with
fewer than 16 elements are judged element by element against 2^-10 * (sum |x||w| + |bias| + |residual|) instead: with
a handful of outputs max|ref| can be one cancelling dot product, which says nothing about the rounding of its terms
(TF32 keeps 10 mantissa bits, so each product is off by at most 2^-10 of its magnitude).
"""
import numpy as np
import pytest
import torch

import convcases as cc
from oracle import oracle
from tracea_b200 import ffi, ops

pytestmark = pytest.mark.gpu

TD = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
EPIS = ["", "bias", "relu", "bias+relu", "bias+silu", "gelu", "residual", "residual+relu", "bias+residual+relu",
        "bias+residual"]


def dev(a, dt):
    return torch.from_numpy(np.ascontiguousarray(a)).to(TD[dt]).cuda()


def split(epi):
    o = [x for x in epi.split("+") if x]
    return "bias" in o, "residual" in o, next((x for x in o if x in ("relu", "silu", "gelu")), "none")


def one_case(rng):
    kind = str(rng.choice(["conv", "convt", "gemm"]))
    dt = str(rng.choice(["bf16", "f16", "f32"]))
    epi = str(rng.choice(EPIS))
    ub, ur, act = split(epi)
    if kind == "conv":
        N, C = int(rng.integers(1, 5)), int(rng.choice([3, 8, 16, 20, 32, 64, 96, 128]))
        K = int(rng.choice([5, 8, 24, 64, 72, 128, 200, 256, 320]))
        R, S = int(rng.integers(1, 6)), int(rng.integers(1, 6))
        sh, sw = int(rng.integers(1, 4)), int(rng.integers(1, 4))
        ph, pw = int(rng.integers(0, R + 1)), int(rng.integers(0, S + 1))
        dh, dw = int(rng.integers(1, 3)), int(rng.integers(1, 3))
        H = int(rng.integers(max(1, dh * (R - 1) + 1 - 2 * ph), 30))
        W = int(rng.integers(max(1, dw * (S - 1) + 1 - 2 * pw), 30))
        x = rng.standard_normal((N, C, H, W)).astype(np.float32)
        w = (rng.standard_normal((K, C, R, S)) * (C * R * S) ** -0.5).astype(np.float32)
        b = rng.standard_normal(K).astype(np.float32) * 0.1
        r = rng.standard_normal(oracle.out_shape(x.shape, w.shape, (sh, sw), (ph, pw), (dh, dw))).astype(np.float32)
        cl_x, cl_w, cl_o = (bool(v) for v in rng.integers(0, 2, 3))
        tx, tw = dev(x, dt), dev(w, dt)
        if cl_x:
            tx = tx.contiguous(memory_format=torch.channels_last)
        if cl_w:
            tw = tw.contiguous(memory_format=torch.channels_last)
        tr = dev(r, dt) if ur else None
        if ur and cl_o:
            tr = tr.contiguous(memory_format=torch.channels_last)
        got = ops.conv2d_nchw(tx, tw, torch.from_numpy(b).cuda() if ub else None, tr, (sh, sw), (ph, pw), (dh, dw), 1,
                              epi or None, channels_last_out=cl_o)
        want = oracle.conv2d(cc.round_to(x, dt), cc.round_to(w, dt), b if ub else None,
                             cc.round_to(r, dt) if ur else None, (sh, sw), (ph, pw), (dh, dw), act)
        desc = ("conv", dt, epi, N, C, H, W, K, R, S, sh, sw, ph, pw, dh, dw, cl_x, cl_w, cl_o)
    elif kind == "convt":
        N, C = int(rng.integers(1, 4)), int(rng.choice([3, 8, 16, 32, 64, 128]))
        K = int(rng.choice([5, 8, 24, 64, 128, 136]))
        R, S = int(rng.integers(1, 6)), int(rng.integers(1, 6))
        sh, sw = int(rng.integers(1, 4)), int(rng.integers(1, 4))
        ph, pw = int(rng.integers(0, R + 1)), int(rng.integers(0, S + 1))
        oh, ow = int(rng.integers(0, sh)), int(rng.integers(0, sw))
        H, W = int(rng.integers(1, 14)), int(rng.integers(1, 14))
        Ho, Wo = (H - 1) * sh - 2 * ph + R + oh, (W - 1) * sw - 2 * pw + S + ow
        if Ho <= 0 or Wo <= 0:
            return None
        x = rng.standard_normal((N, H, W, C)).astype(np.float32)
        w = (rng.standard_normal((K, R, S, C)) * (C * R * S) ** -0.5).astype(np.float32)
        b = rng.standard_normal(K).astype(np.float32) * 0.1
        r = rng.standard_normal((N, Ho, Wo, K)).astype(np.float32)
        got = ops.conv_transpose2d(dev(x, dt), dev(w, dt), torch.from_numpy(b).cuda() if ub else None,
                                   dev(r, dt) if ur else None, epi or None, (sh, sw), (ph, pw), (oh, ow))
        want = oracle.conv_transpose2d(cc.round_to(x, dt), cc.round_to(w, dt), b if ub else None,
                                       cc.round_to(r, dt) if ur else None, (sh, sw), (ph, pw), (oh, ow), act)
        desc = ("convt", dt, epi, N, H, W, C, K, R, S, sh, sw, ph, pw, oh, ow)
    else:
        M = int(rng.choice([1, 7, 100, 129, 300, 700]))
        Kd = int(rng.choice([8, 20, 64, 100, 256, 520]))
        Nn = int(rng.choice([1, 9, 64, 200, 256, 1000, 2312]))
        a = rng.standard_normal((M, Kd)).astype(np.float32)
        bm = (rng.standard_normal((Kd, Nn)) * Kd ** -0.5).astype(np.float32)
        b = rng.standard_normal(Nn).astype(np.float32) * 0.1
        r = rng.standard_normal((M, Nn)).astype(np.float32)
        ta, tb = dev(a, dt), dev(bm, dt)
        if rng.integers(0, 2):
            tb = tb.t().contiguous().t()
        if rng.integers(0, 2):
            ta = ta.t().contiguous().t()
        got = ops.gemm(ta, tb, torch.from_numpy(b).cuda() if ub else None, epi or None, dev(r, dt) if ur else None)
        want = oracle.gemm(cc.round_to(a, dt), cc.round_to(bm, dt), b if ub else None,
                           cc.round_to(r, dt) if ur else None, act)
        desc = ("gemm", dt, epi, M, Kd, Nn)
    torch.cuda.synchronize()
    if dt == "f32" and want.size < 16:
        # magnitude of the terms behind every output: the same operator on absolute values, no epilogue
        if kind == "conv":
            mag = oracle.conv2d(np.abs(x), np.abs(w), None, None, (sh, sw), (ph, pw), (dh, dw))
        elif kind == "convt":
            mag = oracle.conv_transpose2d(np.abs(x), np.abs(w), None, None, (sh, sw), (ph, pw), (oh, ow))
        else:
            mag = oracle.gemm(np.abs(a), np.abs(bm))
        mag = mag + (np.abs(b).reshape([1, -1, 1, 1] if kind == "conv" else [-1]) if ub else 0.0) + (np.abs(r) if ur else 0.0)
        diff = np.abs(got.float().cpu().numpy().astype(np.float64) - want)
        # GELU's slope reaches 1.13; 1.25 leaves room for the fp32 rounding of the epilogue itself
        err = float((diff / (1.25 * 2.0 ** -10 * mag + 1e-30)).max())
        return desc, err, 1.0
    err = cc.rel_err(got.float().cpu().numpy(), cc.round_to(np.ascontiguousarray(want), dt))
    return desc, err, cc.tol_for(dt)


def one_big_case(rng):
    """A layer of ResNet size: C and K_out up to 2304, up to ~200 k output pixels -- several waves of tiles, panels of
    column tiles, CTA pairs, K-splits."""
    while True:
        dt = str(rng.choice(["bf16", "f16"]))
        epi = str(rng.choice(["", "bias+relu", "bias+residual+relu", "bias+silu", "residual"]))
        ub, ur, act = split(epi)
        C = int(rng.choice([64, 128, 192, 256, 512, 1024]))
        K = int(rng.choice([64, 128, 256, 384, 512, 1024, 2048, 2304]))
        R = int(rng.choice([1, 1, 3, 3, 2, 5]))
        s = int(rng.choice([1, 1, 2]))
        p = int(rng.integers(0, R // 2 + 1))
        H = int(rng.choice([7, 14, 28, 56]))
        N = int(rng.choice([1, 3, 8, 17, 32, 64]))
        if N * H * H * C * R * R * K > 6e11 or N * H * H * max(C, K) > 6e7 or H + 2 * p < R:
            continue
        break
    x = np.abs(rng.standard_normal((N, C, H, H))).astype(np.float32)
    w = (rng.standard_normal((K, C, R, R)) * (2.0 / (C * R * R)) ** 0.5).astype(np.float32)
    b = rng.standard_normal(K).astype(np.float32) * 0.05
    r = rng.standard_normal(oracle.out_shape(x.shape, w.shape, s, p, 1)).astype(np.float32)
    cl = lambda t: t.contiguous(memory_format=torch.channels_last)
    got = ops.conv2d_nchw(cl(dev(x, dt)), cl(dev(w, dt)), torch.from_numpy(b).cuda() if ub else None,
                          cl(dev(r, dt)) if ur else None, s, p, 1, 1, epi or None)
    torch.cuda.synchronize()
    want = oracle.conv2d_gemm(cc.channels_last(cc.round_to(x, dt)), cc.round_to(w, dt), b if ub else None,
                              cc.channels_last(cc.round_to(r, dt)) if ur else None, s, p, 1, act)
    err = cc.rel_err(got.float().cpu().numpy(), cc.round_to(np.ascontiguousarray(want), dt))
    return (dt, epi, N, C, H, K, R, s, p), err, cc.TOL_16BIT


def test_resnet_sized_random_layers_match_the_oracle():
    rng = np.random.default_rng(404)
    bad = []
    for _ in range(60):
        desc, err, tol = one_big_case(rng)
        if not err <= tol:
            bad.append((desc, err))
    assert ffi.load().tracea_b200_device_status(0) == 0
    assert not bad, bad[:5]


@pytest.mark.parametrize("seed", [101, 202, 303])
def test_random_cases_match_the_oracle(seed):
    rng = np.random.default_rng(seed)
    bad, done = [], 0
    for _ in range(250):
        res = one_case(rng)
        if res is None:
            continue
        done += 1
        desc, err, tol = res
        if not err <= tol:
            bad.append((desc, err))
    assert ffi.load().tracea_b200_device_status(0) == 0
    assert done >= 200
    assert not bad, bad[:5]

"""Seeded random parity sweep: conv2d, conv_transpose2d and gemm over shapes, strides, paddings, dilations, dtypes,
memory layouts and every epilogue kind, each case against the CPU oracle through the C ABI.

Tolerances as everywhere: 1e-2 * max|ref| (fp16 / bf16), 5e-3 * max|ref| (fp32 computed as TF32); outputs with fewer
than 16 elements are skipped for fp32 because a single cancelling dot product makes max|ref| meaningless as a scale.
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
        return None
    err = cc.rel_err(got.float().cpu().numpy(), cc.round_to(np.ascontiguousarray(want), dt))
    return desc, err, cc.tol_for(dt)


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

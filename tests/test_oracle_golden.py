"""The CPU oracle against the committed known-answer fixtures (tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest

import convcases as cc
from golden.make_golden import CASES
from oracle import oracle

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "conv2d_golden.npz"))


def _epi(spec):
    ops = [o for o in spec[10].split("+") if o]
    act = next((o for o in ops if o in ("relu", "silu", "gelu")), "none")
    return "bias" in ops, "residual" in ops, act


@pytest.mark.parametrize("name", sorted(CASES))
def test_scalar_oracle_matches_golden(name):
    spec = CASES[name]
    x, w, b, res, ref = (GOLDEN[name + "/" + k] for k in ("x", "w", "b", "res", "out"))
    use_b, use_r, act = _epi(spec)
    out = oracle.conv2d(x, w, b if use_b else None, res if use_r else None, spec[7], spec[8], spec[9], act)
    assert out.shape == ref.shape
    assert cc.rel_err(out, ref) < 2e-6


@pytest.mark.parametrize("name", sorted(CASES))
def test_scalar_oracle_reads_channels_last_in_place(name):
    spec = CASES[name]
    x, w, b, res, ref = (GOLDEN[name + "/" + k] for k in ("x", "w", "b", "res", "out"))
    use_b, use_r, act = _epi(spec)
    out = oracle.conv2d(cc.channels_last(x), cc.channels_last(w), b if use_b else None,
                        cc.channels_last(res) if use_r else None, spec[7], spec[8], spec[9], act,
                        channels_last_out=True)
    assert out.strides[1] == 4  # channel is the innermost axis in memory
    assert cc.rel_err(out, ref) < 2e-6


@pytest.mark.parametrize("name", sorted(CASES))
def test_gemm_oracle_matches_golden(name):
    spec = CASES[name]
    x, w, b, res, ref = (GOLDEN[name + "/" + k] for k in ("x", "w", "b", "res", "out"))
    use_b, use_r, act = _epi(spec)
    out = oracle.conv2d_gemm(cc.channels_last(x), w, b if use_b else None, res if use_r else None,
                             spec[7], spec[8], spec[9], act)
    assert cc.rel_err(out, ref) < 2e-6


def test_gemm_oracle_rejects_nchw_memory():
    x = cc.uniform((1, 8, 4, 4), 0, "t/x")
    w = cc.uniform((4, 8, 1, 1), 0, "t/w")
    with pytest.raises(ValueError):
        oracle.conv2d_gemm(x, w)


def test_points_oracle_matches_full_tensor():
    name = "strided_bias_silu"
    spec = CASES[name]
    x, w, b, ref = (GOLDEN[name + "/" + k] for k in ("x", "w", "b", "out"))
    rng = np.random.default_rng(1)
    idx = np.stack([rng.integers(0, s, 200) for s in ref.shape], axis=1)
    vals = oracle.conv2d_points(x, w, idx, b, None, spec[7], spec[8], spec[9], "silu")
    want = ref[idx[:, 0], idx[:, 1], idx[:, 2], idx[:, 3]]
    assert np.abs(vals - want).max() < 2e-6 * np.abs(ref).max()


def test_config1_full_size_digest():
    """Benchmark config 1 at its full size, against the digest written by make_golden.py."""
    dig = np.load(os.path.join(os.path.dirname(__file__), "golden", "conv2d_cfg1_digest.npz"))
    x = cc.uniform((1, 64, 56, 56), 0, "cfg1/x")
    w = cc.uniform((64, 64, 3, 3), 0, "cfg1/w")
    b = cc.normal((64,), 0, "cfg1/b", 0.1)
    sums = np.array([x.astype(np.float64).sum(), w.astype(np.float64).sum(), b.astype(np.float64).sum()])
    if not np.allclose(sums, dig["input_checksums"], rtol=0, atol=1e-9):
        pytest.skip("numpy's Philox stream differs from the one the digest was made with")
    out = oracle.conv2d(x, w, b, None, 1, 1, 1, "relu")
    scale = float(dig["out_absmax"][0])
    assert np.abs(out.reshape(-1)[::7] - dig["out_every7"]).max() < 2e-6 * scale
    assert np.abs(out.astype(np.float64).sum(axis=(0, 2, 3)) - dig["out_channel_sums"]).max() < 1e-3
    out_g = oracle.conv2d_gemm(cc.channels_last(x), w, b, None, 1, 1, 1, "relu")
    assert cc.rel_err(out_g, out) < 2e-6


def test_output_extent_formula():
    # (in + 2 pad - dil (filt - 1) - 1) / stride + 1, src/emitter/cuda/conv.rs:40-41
    assert oracle.out_shape((1, 3, 224, 224), (64, 3, 7, 7), 2, 3) == (1, 64, 112, 112)
    assert oracle.out_shape((1, 64, 224, 224), (128, 64, 3, 3), 1, 0) == (1, 128, 222, 222)
    assert oracle.out_shape((2, 8, 11, 13), (5, 8, 3, 2), (2, 1), (2, 0), (2, 3)) == (2, 5, 6, 10)


def test_rounding_helpers():
    a = np.array([1.0, 1.00390625, 1.005859375, -3.1415927, 65504.0, 1e-8], np.float32)
    import torch
    want = torch.from_numpy(a).to(torch.bfloat16).float().numpy()
    assert np.array_equal(cc.round_to(a, "bf16"), want)
    want16 = torch.from_numpy(a).to(torch.float16).float().numpy()
    assert np.array_equal(cc.round_to(a, "f16"), want16)

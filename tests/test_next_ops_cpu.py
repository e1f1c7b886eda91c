"""ConvTranspose2d and GEMM, CPU side: the oracle against its golden fixtures, and the validation of the two
entry points (which happens before any device is touched)."""
import os

import numpy as np
import pytest

import convcases as cc
from golden.make_golden_next_ops import CONVT_CASES, GEMM_CASES
from oracle import oracle
from tracea_b200 import ffi

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "next_ops_golden.npz"))


def split_epi(epi):
    ops_ = [o for o in (epi or "").split("+") if o]
    act = next((o for o in ops_ if o in ("relu", "silu", "gelu")), "none")
    return "bias" in ops_, "residual" in ops_, act


@pytest.mark.parametrize("name", sorted(CONVT_CASES))
def test_conv_transpose_oracle_reproduces_the_golden_outputs(name):
    spec = CONVT_CASES[name]
    g = {k: GOLDEN["convt/%s/%s" % (name, k)] for k in ("x", "w", "b", "res", "out")}
    use_b, use_r, act = split_epi(spec[10])
    got = oracle.conv_transpose2d(g["x"], g["w"], g["b"] if use_b else None, g["res"] if use_r else None,
                                  spec[7], spec[8], spec[9], act)
    assert got.shape == g["out"].shape
    assert cc.rel_err(got, g["out"]) <= 2e-6


def test_conv_transpose_oracle_reads_the_reference_kernels_weight_memory():
    """The reference's kernel indexes its weights as [(c*R + r)*S + s][K] (src/emitter/conv_transpose.rs:232-243,
    examples/verify_conv_transpose.rs:38-43): the same values through a strided (K, R, S, C) view."""
    name = "s2_p1_3x3_opad"
    spec = CONVT_CASES[name]
    g = {k: GOLDEN["convt/%s/%s" % (name, k)] for k in ("x", "w", "b", "out")}
    crsk = np.ascontiguousarray(g["w"].transpose(3, 1, 2, 0))          # memory [C][R][S][K]
    view = crsk.transpose(3, 1, 2, 0)                                   # logical (K, R, S, C)
    got = oracle.conv_transpose2d(g["x"], view, g["b"], None, spec[7], spec[8], spec[9], "none")
    assert cc.rel_err(got, g["out"]) <= 2e-6


@pytest.mark.parametrize("name", sorted(GEMM_CASES))
def test_gemm_oracle_reproduces_the_golden_outputs(name):
    g = {k: GOLDEN["gemm/%s/%s" % (name, k)] for k in ("a", "bm", "b", "res", "out")}
    use_b, use_r, act = split_epi(GEMM_CASES[name][3])
    got = oracle.gemm(g["a"], g["bm"], g["b"] if use_b else None, g["res"] if use_r else None, act)
    assert cc.rel_err(got, g["out"]) <= 2e-6
    # a transposed-memory B gives the same values
    bt = np.ascontiguousarray(g["bm"].T).T
    assert np.array_equal(oracle.gemm(g["a"], bt, g["b"] if use_b else None, g["res"] if use_r else None, act), got)


# --------------------------------------------------------------------------- validation (no device needed)
_DT = {np.dtype(np.float32): ffi.DTYPE_FLOAT32, np.dtype(np.float16): ffi.DTYPE_FLOAT16,
       np.dtype(np.int32): ffi.DTYPE_INT32}


def _view(a, device=-1, ptr=None):
    v = ffi.View(a.ctypes.data if ptr is None else ptr, a.shape, [s // a.itemsize for s in a.strides], _DT[a.dtype],
                 device)
    v._keep = a
    return v


@pytest.fixture(scope="module")
def lib():
    return ffi.load()


def test_gemm_validation(lib):
    a, b, c = np.zeros((4, 8), np.float32), np.zeros((8, 6), np.float32), np.zeros((4, 6), np.float32)
    assert ffi.gemm_raw(_view(a, ptr=0), _view(b), None, None, _view(c), check=False) == ffi.INVALID_PARAMS
    assert ffi.last_error() == "Null pointer in input tensors"
    assert ffi.gemm_raw(_view(np.zeros((1, 4, 8), np.float32)), _view(b), None, None, _view(c),
                        check=False) == ffi.INVALID_PARAMS
    assert "2D" in ffi.last_error()
    assert ffi.gemm_raw(_view(a), _view(np.zeros((7, 6), np.float32)), None, None, _view(c),
                        check=False) == ffi.INVALID_PARAMS
    assert "Inner dimension mismatch" in ffi.last_error()
    assert ffi.gemm_raw(_view(a), _view(b), None, None, _view(np.zeros((4, 5), np.float32)),
                        check=False) == ffi.INVALID_PARAMS
    assert "c shape" in ffi.last_error()
    ai = np.zeros((4, 8), np.int32)
    assert ffi.gemm_raw(_view(ai), _view(b), None, None, _view(c), check=False) == ffi.UNSUPPORTED_CONFIG
    bias = np.zeros(5, np.float32)
    assert ffi.gemm_raw(_view(a), _view(b), _view(bias), None, _view(c), ffi.EPILOGUE_BIAS_ADD,
                        check=False) == ffi.INVALID_PARAMS
    assert "tracea_gemm" in ffi.last_error() and "bias" in ffi.last_error()
    # an empty M is a no-op
    assert ffi.gemm_raw(_view(np.zeros((0, 8), np.float32)), _view(b), None, None, _view(np.zeros((0, 6), np.float32)),
                        check=False) == ffi.SUCCESS


def test_conv_transpose_validation(lib):
    x, w = np.zeros((1, 4, 4, 8), np.float32), np.zeros((6, 3, 3, 8), np.float32)
    o = np.zeros((1, 7, 7, 6), np.float32)       # stride 2, pad 1: (4-1)*2 - 2 + 3 = 7
    call = lambda *a, **k: ffi.conv_transpose2d_raw(*a, check=False, **k)
    assert call(_view(x), _view(w), None, None, _view(o, ptr=0), (2, 2), (1, 1)) == ffi.INVALID_PARAMS
    assert call(_view(x), _view(w), None, None, _view(o), (2, 2), (1, 1), groups=2) == ffi.UNSUPPORTED_CONFIG
    assert call(_view(x), _view(w), None, None, _view(o), (2, 2), (1, 1), dilation=(2, 2)) == ffi.UNSUPPORTED_CONFIG
    assert "dilation" in ffi.last_error()
    assert call(_view(x), _view(w), None, None, _view(o), (0, 2), (1, 1)) == ffi.INVALID_PARAMS
    assert call(_view(x), _view(w), None, None, _view(o), (2, 2), (1, 1), (2, 0)) == ffi.INVALID_PARAMS
    assert "output_padding" in ffi.last_error()
    assert call(_view(x), _view(w), None, None, _view(np.zeros((1, 8, 8, 6), np.float32)), (2, 2), (1, 1)) == ffi.INVALID_PARAMS
    assert "expected [1,7,7,6]" in ffi.last_error()
    assert call(_view(x), _view(np.zeros((6, 3, 3, 4), np.float32)), None, None, _view(o), (2, 2), (1, 1)) == ffi.INVALID_PARAMS
    assert "Channel mismatch" in ffi.last_error()
    assert call(_view(x), _view(w), None, None, _view(o, device=0), (2, 2), (1, 1)) == ffi.INVALID_PARAMS
    # an empty batch is a no-op
    assert call(_view(np.zeros((0, 4, 4, 8), np.float32)), _view(w), None, None, _view(np.zeros((0, 7, 7, 6), np.float32)),
                (2, 2), (1, 1)) == ffi.SUCCESS


def test_prepack_validation(lib):
    w = np.zeros((4, 8, 3, 3), np.float32)
    v = _view(w)
    assert lib.tracea_conv2d_prepack_bytes(v.c) == 4 * 8 * 9 * 4
    w3 = np.zeros((4, 3, 3, 3), np.float16)     # 3 channels pad to 8 halves
    assert lib.tracea_conv2d_prepack_bytes(_view(w3).c) == 4 * 8 * 9 * 2
    assert lib.tracea_conv2d_prepack_bytes(_view(np.zeros((4, 8), np.float32)).c) == 0
    import ctypes
    shape, stride = (ctypes.c_uint64 * 4)(), (ctypes.c_int64 * 4)()
    st = lib.tracea_conv2d_prepack(v.c, 16, 4 * 8 * 9 * 4, shape, stride, None)   # host view
    assert st == ffi.INVALID_PARAMS and "device tensors" in ffi.last_error()
    b = np.zeros((8, 6), np.float32)
    assert lib.tracea_gemm_prepack_b_bytes(_view(b).c) == 8 * 6 * 4
    st2 = (ctypes.c_int64 * 2)()
    assert lib.tracea_gemm_prepack_b(_view(b, device=0).c, 16, 10, st2, None) == ffi.INVALID_PARAMS
    assert "needs" in ffi.last_error()


# --------------------------------------------------------------------------- the phase plan (host arithmetic)
def _replay_plan_1d(x, w, stride, pad, opad):
    """x: (H,), w: (R,). Runs the library's per-phase plan as plain stride-1 correlations and scatters the phases."""
    H, R = len(x), len(w)
    Ho = (H - 1) * stride - 2 * pad + R + opad
    out = np.full(Ho, np.nan)
    for ph in ffi.conv_transpose_plan(H, Ho, R, stride, pad):
        if ph["T"] == 0:
            continue
        if ph["a"] < 0:
            taps = np.zeros(1)
        else:
            taps = np.array([w[ph["a"] + stride * (ph["taps"] - 1 - j)] for j in range(ph["taps"])])
        assert ph["in"] >= 1 and ph["pad_lo"] >= 0 and ph["pad_hi"] >= 0 and ph["x_off"] + ph["in"] <= H
        assert ph["T"] == ph["in"] + ph["pad_lo"] + ph["pad_hi"] - (ph["taps"] - 1)
        xp = np.concatenate([np.zeros(ph["pad_lo"]), x[ph["x_off"]:ph["x_off"] + ph["in"]], np.zeros(ph["pad_hi"])])
        vals = np.array([np.dot(xp[t:t + ph["taps"]], taps) for t in range(ph["T"])])
        out[ph["a0"]::stride] = vals
    assert not np.isnan(out).any()          # the phases cover every output exactly
    return out


@pytest.mark.parametrize("H,R,stride,pad,opad", [
    (5, 3, 1, 0, 0), (5, 3, 1, 1, 0), (6, 5, 1, 3, 0), (4, 2, 2, 0, 0), (5, 3, 2, 1, 1), (8, 4, 2, 1, 0),
    (5, 2, 3, 0, 1), (5, 2, 3, 0, 2), (7, 5, 3, 2, 1), (3, 7, 2, 3, 1), (9, 1, 2, 0, 1), (6, 3, 4, 1, 3),
    (2, 6, 5, 2, 4), (10, 4, 2, 3, 0), (1, 3, 2, 1, 1),
])
def test_phase_plan_reproduces_the_transposed_convolution(H, R, stride, pad, opad):
    if (H - 1) * stride - 2 * pad + R + opad <= 0:
        pytest.skip("empty output")
    rng = cc.rng_for(1, "plan/%d/%d/%d/%d/%d" % (H, R, stride, pad, opad))
    x, w = rng.standard_normal(H), rng.standard_normal(R)
    got = _replay_plan_1d(x, w, stride, pad, opad)
    want = oracle.conv_transpose2d(x.astype(np.float32).reshape(1, H, 1, 1), w.astype(np.float32).reshape(1, R, 1, 1),
                                   None, None, (stride, 1), (pad, 0), (opad, 0)).reshape(-1)
    assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max())


def test_phase_plan_rejects_bad_arguments(lib):
    import ctypes
    buf = (ctypes.c_int64 * 16)()
    assert lib.tracea_b200_conv_transpose_plan(4, 8, 3, 0, 0, buf) == -1
    assert lib.tracea_b200_conv_transpose_plan(4, 8, 3, 2, 0, None) == -1

"""tracea_conv2d_noalloc: the variant of tracea_conv2d whose staging memory is a fixed array inside
the library instead of an allocation. It serves callers that cannot go to the CUDA allocator at call
time -- processes whose own arena already owns all free GPU memory, and latency-critical loops that
cannot take an allocation's implicit synchronisation.

The file name sorts last on purpose: if this test fails under `pytest -x`, every other test has
already run. It also passes when run alone in a fresh process (the first call on a device does the
entry point's one-time set-up).
"""
import numpy as np
import pytest
import torch

import convcases as cc
from tracea_b200 import ffi, ops

pytestmark = pytest.mark.gpu


def _call(entry, x, w, b, res, out, stride, pad, kind):
    ffi.conv2d_raw(ops._view(x), ops._view(w), ops._view(b) if b is not None else None,
                   ops._view(res) if res is not None else None, ops._view(out), (stride, stride), (pad, pad), (1, 1), 1,
                   kind, torch.cuda.current_stream().cuda_stream, entry=entry)
    torch.cuda.synchronize()
    return out


CASES = [
    # dtype, N, C, H, W, K, R, stride, pad, epilogue     (x NCHW-contiguous, w OIHW-contiguous: both staged)
    ("f32", 1, 64, 56, 56, 64, 3, 1, 1, "bias+relu"),
    ("bf16", 3, 24, 17, 19, 40, 3, 2, 1, "bias+residual+relu"),
]


def test_noalloc_entry_matches_tracea_conv2d_on_two_calls_in_a_row():
    dt = {"f32": torch.float32, "bf16": torch.bfloat16}
    for dtype, N, C, H, W, K, R, stride, pad, epi in CASES:        # two different calls back to back
        x = torch.from_numpy(cc.uniform((N, C, H, W), 11, "na/x")).to(dt[dtype]).cuda()
        w = torch.from_numpy(cc.kaiming((K, C, R, R), 11, "na/w")).to(dt[dtype]).cuda()
        b = torch.from_numpy(cc.normal((K,), 11, "na/b", 0.1)).cuda()
        ho, wo = (H + 2 * pad - R) // stride + 1, (W + 2 * pad - R) // stride + 1
        res = torch.from_numpy(cc.normal((N, K, ho, wo), 11, "na/r")).to(dt[dtype]).cuda() if "residual" in epi else None
        kind = ops.parse_epilogue(epi, b, res)
        want = _call("tracea_conv2d", x, w, b, res, torch.empty((N, K, ho, wo), dtype=dt[dtype], device="cuda"),
                     stride, pad, kind)
        got = _call("tracea_conv2d_noalloc", x, w, b, res,
                    torch.full((N, K, ho, wo), float("nan"), dtype=dt[dtype], device="cuda"), stride, pad, kind)
        err = cc.rel_err(got.float().cpu().numpy(), want.float().cpu().numpy())
        assert err <= cc.tol_for(dtype), (dtype, err)
    # and the first case once more, after the scratch has held another call's data
    dtype, N, C, H, W, K, R, stride, pad, epi = CASES[0]
    x = torch.from_numpy(cc.uniform((N, C, H, W), 12, "na/x")).cuda()
    w = torch.from_numpy(cc.kaiming((K, C, R, R), 12, "na/w")).cuda()
    b = torch.from_numpy(cc.normal((K,), 12, "na/b", 0.1)).cuda()
    kind = ops.parse_epilogue(epi, b, None)
    want = _call("tracea_conv2d", x, w, b, None, torch.empty((N, K, H, W), device="cuda"), stride, pad, kind)
    got = _call("tracea_conv2d_noalloc", x, w, b, None, torch.empty((N, K, H, W), device="cuda"), stride, pad, kind)
    assert cc.rel_err(got.cpu().numpy(), want.cpu().numpy()) <= cc.TOL_TF32
    assert ffi.load().tracea_b200_device_status(0) == 0


def test_noalloc_entry_rejects_what_does_not_fit_and_host_memory():
    # 1 x 64 x 512 x 512 fp32 needs a 64 MiB channels-last copy: more than the 16 MiB built in
    x = torch.zeros((1, 64, 512, 512), device="cuda")
    w = torch.zeros((8, 64, 1, 1), device="cuda")
    out = torch.empty((1, 8, 512, 512), device="cuda")
    with pytest.raises(ffi.TraceaError) as e:
        _call("tracea_conv2d_noalloc", x, w, None, None, out, 1, 0, ffi.EPILOGUE_IDENTITY)
    assert e.value.status == ffi.UNSUPPORTED_CONFIG and "built-in scratch holds" in e.value.message
    # the same tensor in channels-last memory needs no staging and is accepted
    x_cl = x.contiguous(memory_format=torch.channels_last)
    w_cl = w.contiguous(memory_format=torch.channels_last)
    _call("tracea_conv2d_noalloc", x_cl, w_cl, None, None, out, 1, 0, ffi.EPILOGUE_IDENTITY)
    assert float(out.abs().max()) == 0.0
    # host tensors would have to be staged through an allocation
    hx, hw, ho = np.zeros((1, 8, 4, 4), np.float32), np.zeros((8, 8, 1, 1), np.float32), np.zeros((1, 8, 4, 4), np.float32)
    mk = lambda a: ffi.View(a.ctypes.data, a.shape, [s // 4 for s in a.strides], ffi.DTYPE_FLOAT32, -1)
    st = ffi.conv2d_raw(mk(hx), mk(hw), None, None, mk(ho), check=False, entry="tracea_conv2d_noalloc")
    assert st == ffi.INVALID_PARAMS

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
from oracle import oracle
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
DT = {"f32": torch.float32, "bf16": torch.bfloat16}


def _inputs(case, seed):
    dtype, N, C, H, W, K, R, stride, pad, epi = case
    x = cc.uniform((N, C, H, W), seed, "na/x")
    w = cc.kaiming((K, C, R, R), seed, "na/w")
    b = cc.normal((K,), seed, "na/b", 0.1)
    ho, wo = (H + 2 * pad - R) // stride + 1, (W + 2 * pad - R) // stride + 1
    res = cc.normal((N, K, ho, wo), seed, "na/r") if "residual" in epi else None
    return x, w, b, res, (N, K, ho, wo)


def _oracle(case, x, w, b, res):
    dtype, _, _, _, _, _, _, stride, pad, epi = case
    xr, wr = cc.round_to(x, dtype), cc.round_to(w, dtype)
    rr = cc.round_to(res, dtype) if res is not None else None
    want = oracle.conv2d_gemm(cc.channels_last(xr), wr, b, rr, stride, pad, 1, "relu")
    return cc.round_to(np.ascontiguousarray(want), dtype)


def test_noalloc_entry_matches_tracea_conv2d_and_the_oracle_on_two_calls_in_a_row():
    """Same kernel, same inputs: the two entries must agree bit for bit, and both with the CPU oracle."""
    for seed, case in ((11, CASES[0]), (11, CASES[1]), (12, CASES[0])):   # the last: after the scratch held other data
        dtype, _, _, _, _, _, _, stride, pad, epi = case
        x, w, b, res, oshape = _inputs(case, seed)
        tx, tw = torch.from_numpy(x).to(DT[dtype]).cuda(), torch.from_numpy(w).to(DT[dtype]).cuda()
        tb = torch.from_numpy(b).cuda()
        tr = torch.from_numpy(res).to(DT[dtype]).cuda() if res is not None else None
        kind = ops.parse_epilogue(epi, tb, tr)
        want = _call("tracea_conv2d", tx, tw, tb, tr, torch.empty(oshape, dtype=DT[dtype], device="cuda"), stride, pad,
                     kind)
        got = _call("tracea_conv2d_noalloc", tx, tw, tb, tr,
                    torch.full(oshape, float("nan"), dtype=DT[dtype], device="cuda"), stride, pad, kind)
        assert torch.equal(got, want), (dtype, seed)
        err = cc.rel_err(got.float().cpu().numpy(), _oracle(case, x, w, b, res))
        assert err <= cc.tol_for(dtype), (dtype, err)
    assert ffi.load().tracea_b200_device_status(0) == 0


def test_noalloc_entry_takes_no_memory_from_the_device_or_the_pool():
    """Steady state (the kernels of this shape have run once, so the driver has loaded them): across a call
    the device's free memory does not move and the library's scratch pool hands nothing out."""
    case = CASES[0]
    dtype, _, _, _, _, _, _, stride, pad, epi = case
    x, w, b, res, oshape = _inputs(case, 13)
    tx, tw, tb = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), torch.from_numpy(b).cuda()
    out = torch.empty(oshape, device="cuda")
    kind = ops.parse_epilogue(epi, tb, None)
    _call("tracea_conv2d", tx, tw, tb, None, out, stride, pad, kind)          # brings the pool up
    _call("tracea_conv2d_noalloc", tx, tw, tb, None, out, stride, pad, kind)  # one-time set-up, module loading
    ffi.pool_stats(0, reset_high=True)
    before = ffi.pool_stats(0)
    assert before is not None
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        _call("tracea_conv2d_noalloc", tx, tw, tb, None, out, stride, pad, kind)
    free_after, _ = torch.cuda.mem_get_info()
    after = ffi.pool_stats(0)
    assert free_after == free_before
    assert after["used"] == before["used"] and after["reserved"] == before["reserved"]
    assert after["used_high"] <= before["used"]          # nothing was handed out since the reset
    # the allocating entry on the same inputs does go to the pool (the counter is live)
    _call("tracea_conv2d", tx, tw, tb, None, out, stride, pad, kind)
    assert ffi.pool_stats(0)["used_high"] > before["used"]


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

"""The kernels' failure path, exercised without faulting, trapping or hanging anything: every wait inside them is
bounded, and a wait that runs out makes its role record a code, the CTA unwind through its normal teardown (copies
drained, TMEM freed) and the kernel return. The library's test hooks shorten the limit of a wait and make the TMA
producer go silent after two pipeline stages, so the MMA issuer's wait for the third stage runs out.

The reference has nothing to compare with: its kernels wait without limit (src/backend/cuda/primitives.rs:70-121).
"""
import numpy as np
import pytest
import torch

import convcases as cc
from oracle import oracle
from tracea_b200 import ffi, ops

pytestmark = pytest.mark.gpu

ERR_MMA_WAIT_FULL = 2     # conv2d_sm100.cuh: the MMA issuer never saw a stage's bytes land

CASES = {
    # name: (N, C, H, K, R, pad, kernel kind expected, stride)
    "single_cta": (8, 64, 28, 128, 3, 1, ffi.KERNEL_GENERAL, 1),          # 128-wide tiles, one CTA per tile
    "cta_pair": (8, 256, 14, 256, 3, 1, ffi.KERNEL_GENERAL, 1),           # 256 x 256 tiles over two SMs (cluster of 2)
    "resident_filter": (64, 64, 56, 64, 3, 1, ffi.KERNEL_RESIDENT_FILTER, 1),   # every CTA pair gets three windows or more
    "row_band": (48, 3, (56, 224), 64, 7, 3, ffi.KERNEL_ROW_BAND, 2),     # RGB stem rows: every CTA gets four bands or more
}


def _tensors(name):
    N, C, H, K, R, pad, _, stride = CASES[name]
    H, W = H if isinstance(H, tuple) else (H, H)
    x = cc.normal((N, C, H, W), 21, "fail/x")
    w = cc.kaiming((K, C, R, R), 21, "fail/w")
    b = cc.normal((K,), 21, "fail/b", 0.1)
    cl = lambda a: torch.from_numpy(a).to(torch.bfloat16).cuda().contiguous(memory_format=torch.channels_last)
    return x, w, b, cl(x), cl(w), torch.from_numpy(b).cuda(), pad, stride


def _check_ok(x, w, b, tx, tw, tb, pad, stride=1):
    got = ops.conv2d_nchw(tx, tw, tb, None, stride, pad, 1, 1, "bias+relu")
    torch.cuda.synchronize()
    want = oracle.conv2d_gemm(cc.channels_last(cc.round_to(x, "bf16")), cc.round_to(w, "bf16"), b, None, stride, pad, 1, "relu")
    assert cc.rel_err(got.float().cpu().numpy(), cc.round_to(np.ascontiguousarray(want), "bf16")) <= cc.TOL_16BIT


@pytest.mark.parametrize("name", sorted(CASES))
def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable(name):
    lib = ffi.load()
    x, w, b, tx, tw, tb, pad, stride = _tensors(name)
    _check_ok(x, w, b, tx, tw, tb, pad, stride)              # warm: kernels loaded, results right
    assert lib.tracea_b200_device_status(0) == 0
    before = ffi.launch_count_of(CASES[name][6])
    try:
        lib.tracea_b200_test_hooks(400000, 2)                # ~0.2 ms per wait; producers stop after two stages
        ops.conv2d_nchw(tx, tw, tb, None, stride, pad, 1, 1, "bias+relu")   # the launch itself succeeds: the call is asynchronous
        torch.cuda.synchronize()                             # and the kernel ends by itself
    finally:
        lib.tracea_b200_test_hooks(0, -1)
    assert ffi.launch_count_of(CASES[name][6]) == before + 1
    assert lib.tracea_b200_device_status(0) == ERR_MMA_WAIT_FULL      # read and cleared
    assert lib.tracea_b200_device_status(0) == 0
    _check_ok(x, w, b, tx, tw, tb, pad, stride)              # same context, same stream: the next call is fine


def test_an_unread_kernel_error_fails_the_next_call_once():
    lib = ffi.load()
    x, w, b, tx, tw, tb, pad, _ = _tensors("single_cta")
    try:
        lib.tracea_b200_test_hooks(400000, 2)
        ops.conv2d_nchw(tx, tw, tb, None, 1, pad, 1, 1, "bias+relu")
        torch.cuda.synchronize()
    finally:
        lib.tracea_b200_test_hooks(0, -1)
    with pytest.raises(ffi.TraceaError) as e:                # tracea_conv2d looks at the status word on the way in
        ops.conv2d_nchw(tx, tw, tb, None, 1, pad, 1, 1, "bias+relu")
    assert e.value.status == ffi.CUDA_ERROR and "gave up a bounded wait (code 2" in e.value.message
    _check_ok(x, w, b, tx, tw, tb, pad)
    assert lib.tracea_b200_device_status(0) == 0

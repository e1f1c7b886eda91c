"""One process, one host thread per GPU, `device_id = g` in the views (how a caller shards a batch over the GPUs of
a box without a process per GPU): the threads run concurrently -- the library keeps no process-wide lock on the call
path -- and every device returns the bits the single-device run returns. Skipped on a box with one GPU."""
import threading

import pytest
import torch

import convcases as cc
from tracea_b200 import ffi, ops, shard

pytestmark = pytest.mark.gpu


def _layer(dev, x, w, b, res):
    cl = lambda a: torch.from_numpy(a).to(torch.bfloat16).to(dev).contiguous(memory_format=torch.channels_last)
    return cl(x), cl(w), torch.from_numpy(b).to(dev), cl(res)


def test_two_threads_drive_two_devices_with_identical_results():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    n = 64
    x = cc.normal((n, 256, 14, 14), 31, "md/x")
    w = cc.kaiming((256, 256, 3, 3), 31, "md/w")
    b = cc.normal((256,), 31, "md/b", 0.05)
    res = cc.normal((n, 256, 14, 14), 31, "md/r")
    # reference: the whole batch on device 0, one thread
    tx, tw, tb, tr = _layer("cuda:0", x, w, b, res)
    with torch.cuda.device(0):
        want = ops.conv2d_nchw(tx, tw, tb, tr, 1, 1, 1, 1, "bias+residual+relu")
        torch.cuda.synchronize(0)
    world = 2
    outs, errors = [None] * world, []

    def worker(g):
        try:
            a, e = shard.shard_range(n, g, world)
            dev = "cuda:%d" % g
            gx, gw, gb, gr = _layer(dev, x[a:e], w, b, res[a:e])
            with torch.cuda.device(g):
                for _ in range(20):                      # many calls, so that the two threads really overlap
                    out = ops.conv2d_nchw(gx, gw, gb, gr, 1, 1, 1, 1, "bias+residual+relu")
                torch.cuda.synchronize(g)
            assert ffi.load().tracea_b200_device_status(g) == 0
            outs[g] = out.cpu()
        except Exception as exc:   # surfaced in the main thread
            errors.append((g, exc))

    threads = [threading.Thread(target=worker, args=(g,)) for g in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert torch.equal(torch.cat(outs), want.cpu())

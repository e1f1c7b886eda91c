"""One bf16 GEMM through tracea_gemm, a few times, for profiling: `python -m tracea_b200.gemm_example [M K N [iters]]`.
b is held as [N][K] memory (the layout a Linear layer's weight has) and read in place."""
import sys

import torch

from . import ffi, ops


def main(argv):
    m, k, n = (int(v) for v in argv[:3]) if len(argv) >= 3 else (8192, 8192, 8192)
    iters = int(argv[3]) if len(argv) >= 4 else 4
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn((m, k), device="cuda", dtype=torch.bfloat16, generator=g)
    bt = torch.randn((n, k), device="cuda", dtype=torch.bfloat16, generator=g)
    c = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
    va, vb, vc = ops._view(a), ops._view(bt.t()), ops._view(c)
    for _ in range(iters):
        ffi.gemm_raw(va, vb, None, None, vc, ffi.EPILOGUE_IDENTITY, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    status = ffi.load().tracea_b200_device_status(0)
    print("tracea_gemm %dx%dx%d x%d: device status %d, c[0,0] = %.4f" % (m, k, n, iters, status, float(c[0, 0])))
    return 0 if status == 0 else 1


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))

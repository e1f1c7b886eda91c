"""One bf16 transposed convolution through tracea_conv_transpose2d, a few times, for profiling:
`python -m tracea_b200.conv_transpose_example [N H W C K R stride pad [iters]]` (x is N,H,W,C; w is K,R,R,C)."""
import sys

import torch

from . import ffi, ops


def main(argv):
    n, h, w, c, k, r, stride, pad = (int(v) for v in argv[:8]) if len(argv) >= 8 else (128, 32, 32, 256, 128, 4, 2, 1)
    iters = int(argv[8]) if len(argv) >= 9 else 3
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((n, h, w, c), device="cuda", dtype=torch.bfloat16, generator=g)
    wt = torch.randn((k, r, r, c), device="cuda", dtype=torch.bfloat16, generator=g) * (c * r * r) ** -0.5
    ho, wo = (h - 1) * stride - 2 * pad + r, (w - 1) * stride - 2 * pad + r
    y = torch.empty((n, ho, wo, k), device="cuda", dtype=torch.bfloat16)
    vx, vw, vy = ops._view(x), ops._view(wt), ops._view(y)
    before = ffi.load().tracea_b200_launch_count()
    for _ in range(iters):
        ffi.conv_transpose2d_raw(vx, vw, None, None, vy, (stride, stride), (pad, pad), (0, 0), (1, 1), 1,
                                 ffi.EPILOGUE_IDENTITY, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    status = ffi.load().tracea_b200_device_status(0)
    launches = ffi.load().tracea_b200_launch_count() - before
    print("tracea_conv_transpose2d x[%d,%d,%d,%d] w[%d,%d,%d,%d] /%d p%d x%d: %d kernel launches, device status %d, "
          "y[0,0,0,0] = %.4f" % (n, h, w, c, k, r, r, c, stride, pad, iters, launches, status, float(y[0, 0, 0, 0])))
    return 0 if status == 0 else 1


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))

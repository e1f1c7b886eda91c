"""One bf16 convolution layer through tracea_conv2d, a few times, for profiling:
`python -m tracea_b200.conv_example N C H K R stride pad [epilogue [iters]]` (square images and filters, channels-last
tensors, e.g. `256 64 56 64 3 1 1 bias+relu` for the ResNet-50 3x3 64->64 layer)."""
import sys

import torch

from . import ffi, ops


def main(argv):
    n, c, h, k, r, stride, pad = (int(v) for v in argv[:7]) if len(argv) >= 7 else (256, 64, 56, 64, 3, 1, 1)
    epilogue = argv[7] if len(argv) >= 8 else "bias+relu"
    iters = int(argv[8]) if len(argv) >= 9 else 4
    g = torch.Generator(device="cuda").manual_seed(0)
    cl = torch.channels_last
    x = torch.randn((n, c, h, h), device="cuda", dtype=torch.bfloat16, generator=g).abs_().contiguous(memory_format=cl)
    w = (torch.randn((k, c, r, r), device="cuda", dtype=torch.bfloat16, generator=g) * (2.0 / (c * r * r)) ** 0.5
         ).contiguous(memory_format=cl)
    bias = torch.randn((k,), device="cuda", generator=g) * 0.05
    ho = (h + 2 * pad - r) // stride + 1
    res = torch.randn((n, k, ho, ho), device="cuda", dtype=torch.bfloat16, generator=g).contiguous(memory_format=cl)
    out = torch.empty((n, k, ho, ho), device="cuda", dtype=torch.bfloat16).contiguous(memory_format=cl)
    kind = ops.parse_epilogue(epilogue or None, bias, res)
    use_res = "residual" in epilogue
    for _ in range(iters):
        ops.conv2d_into(x, w, out, bias if "bias" in epilogue else None, res if use_res else None, stride, pad, 1, 1, kind)
    torch.cuda.synchronize()
    status = ffi.load().tracea_b200_device_status(0)
    flops = 2.0 * n * ho * ho * k * c * r * r
    print("tracea_conv2d x[%d,%d,%d,%d] w[%d,%d,%d,%d] /%d p%d %s x%d: %.2f GFLOP per call, device status %d" % (
        n, c, h, h, k, c, r, r, stride, pad, epilogue, iters, flops / 1e9, status))
    return 0 if status == 0 else 1


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))

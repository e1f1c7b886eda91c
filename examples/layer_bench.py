#!/usr/bin/env python
"""Times ONE operator through the C ABI on the current GPU -- the counterpart of the reference's per-layer drivers
(examples/conv_bench.rs, examples/resnet_bench.rs:28-110: build a layer, warm up, launch, report TFLOP/s).

    python examples/layer_bench.py conv N C H K R STRIDE PAD [--epilogue bias+relu] [--dtype bf16] [--nchw]
    python examples/layer_bench.py gemm M N K
    python examples/layer_bench.py conv-transpose N H C K R STRIDE PAD
    python examples/layer_bench.py preset resnet50-3x3-64        # the reference's benchmark layer (batch 64)

Square images and filters, channels-last tensors unless --nchw. `--iters` timed launches between two CUDA events
after `--warmup` untimed ones, over `--sets` rotating operand sets (so that no launch finds its inputs in L2);
`--launch-only` skips the timing and just issues the launches (what a profiler run wants). FLOPs follow the reference's
convention 2*M*K_out*(C*R*S) (src/optimizer/benchmark.rs:458-469).
"""
import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PRESETS = {
    # src/optimizer/benchmark.rs:474-509 and examples/resnet_bench.rs:28-47
    "resnet50-3x3-64": ("conv", [64, 64, 56, 64, 3, 1, 1]),
    "resnet50-3x3-64-b32": ("conv", [32, 64, 56, 64, 3, 1, 1]),
    "resnet50-1x1-64-256": ("conv", [64, 64, 56, 256, 1, 1, 0]),
    "resnet50-stage3-3x3": ("conv", [256, 256, 14, 256, 3, 1, 1]),
}


def build_parser():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("op", choices=["conv", "gemm", "conv-transpose", "preset"])
    ap.add_argument("dims", nargs="+", help="operator dimensions (see above), or the preset's name")
    ap.add_argument("--epilogue", default="bias+relu")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f16", "f32"])
    ap.add_argument("--nchw", action="store_true", help="NCHW / OIHW contiguous tensors (the layout adapters run too)")
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--sets", type=int, default=3)
    ap.add_argument("--launch-only", action="store_true")
    return ap


def parse(argv):
    """Returns (op, dims, args) with presets expanded and the dimension count checked."""
    args = build_parser().parse_args(argv)
    op, dims = args.op, args.dims
    if op == "preset":
        if len(dims) != 1 or dims[0] not in PRESETS:
            raise SystemExit("unknown preset %r (known: %s)" % (dims, ", ".join(sorted(PRESETS))))
        op, dims = PRESETS[dims[0]]
    want = {"conv": 7, "gemm": 3, "conv-transpose": 7}[op]
    if len(dims) != want:
        raise SystemExit("%s takes %d dimensions, got %d" % (op, want, len(dims)))
    return op, [int(d) for d in dims], args


def main(argv=None):
    op, dims, args = parse(sys.argv[1:] if argv is None else argv)
    import torch
    from tracea_b200 import ffi, ops
    dt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[args.dtype]
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    cl = (lambda t: t) if args.nchw else (lambda t: t.contiguous(memory_format=torch.channels_last))
    rnd = lambda *shape: torch.randn(shape, device=dev, generator=g)
    calls = []
    if op == "conv":
        n, c, h, k, r, stride, pad = dims
        ho = (h + 2 * pad - r) // stride + 1
        flops = 2.0 * n * ho * ho * k * c * r * r
        w = cl((rnd(k, c, r, r) * (2.0 / (c * r * r)) ** 0.5).to(dt))
        bias = rnd(k) * 0.05
        for _ in range(args.sets):
            x = cl(rnd(n, c, h, h).abs_().to(dt))
            res = cl(rnd(n, k, ho, ho).to(dt)) if "residual" in args.epilogue else None
            out = cl(torch.empty((n, k, ho, ho), device=dev, dtype=dt))
            kind = ops.parse_epilogue(args.epilogue or None, bias, res)
            b = bias if "bias" in args.epilogue else None
            calls.append(lambda x=x, res=res, out=out, kind=kind, b=b: ops.conv2d_into(x, w, out, b, res, stride, pad, 1, 1, kind))
        what = "conv2d x[%d,%d,%d,%d] w[%d,%d,%d,%d] /%d p%d %s %s%s" % (n, c, h, h, k, c, r, r, stride, pad, args.epilogue,
                                                                         args.dtype, " nchw" if args.nchw else "")
    elif op == "gemm":
        m, n, k = dims
        flops = 2.0 * m * n * k
        bt = rnd(n, k).to(dt)                    # [N][K] memory: b (K, N) with strides (1, K), read in place
        stream = torch.cuda.current_stream().cuda_stream
        for _ in range(args.sets):
            a, c = rnd(m, k).to(dt), torch.empty((m, n), device=dev, dtype=dt)
            va, vb, vc = ops._view(a), ops._view(bt.t()), ops._view(c)
            calls.append(lambda va=va, vb=vb, vc=vc, keep=(a, c): ffi.gemm_raw(va, vb, None, None, vc,
                                                                               ffi.EPILOGUE_IDENTITY, stream))
        what = "gemm %d x %d x %d %s" % (m, n, k, args.dtype)
    else:
        n, h, c, k, r, stride, pad = dims
        ho = (h - 1) * stride - 2 * pad + r
        flops = 2.0 * n * h * h * c * k * r * r
        w = (rnd(k, r, r, c) * (c * r * r) ** -0.5).to(dt)
        stream = torch.cuda.current_stream().cuda_stream
        vw = ops._view(w)
        for _ in range(args.sets):
            x, y = rnd(n, h, h, c).to(dt), torch.empty((n, ho, ho, k), device=dev, dtype=dt)
            vx, vy = ops._view(x), ops._view(y)
            calls.append(lambda vx=vx, vy=vy, keep=(x, y): ffi.conv_transpose2d_raw(
                vx, vw, None, None, vy, (stride, stride), (pad, pad), (0, 0), (1, 1), 1, ffi.EPILOGUE_IDENTITY, stream))
        what = "conv_transpose2d x[%d,%d,%d,%d] w[%d,%d,%d,%d] /%d p%d %s" % (n, h, h, c, k, r, r, c, stride, pad, args.dtype)
    lib = ffi.load()
    for i in range(args.warmup):
        calls[i % len(calls)]()
    torch.cuda.synchronize()
    if args.launch_only:
        for i in range(args.iters):
            calls[i % len(calls)]()
        torch.cuda.synchronize()
        print("%s: %d launches issued, device status %d" % (what, args.iters, lib.tracea_b200_device_status(0)))
        return 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    before = lib.tracea_b200_launch_count()
    e0.record()
    for i in range(args.iters):
        calls[i % len(calls)]()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / args.iters * 1e3
    status = lib.tracea_b200_device_status(0)
    print("%s: %.1f us per call, %.1f TFLOP/s, %d kernel launch(es) per call, device status %d" % (
        what, us, flops / us / 1e6, (lib.tracea_b200_launch_count() - before) // args.iters, status))
    return 0 if status == 0 else 1


if __name__ == "__main__":
    sys.exit(main())

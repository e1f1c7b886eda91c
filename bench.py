#!/usr/bin/env python
"""Benchmark of the Conv2d hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (one "step"): the ResNet-50 stage-3 bottleneck block in bf16 at 256 images per GPU --
1x1 1024->256 +bias+ReLU, 3x3 256->256 pad 1 +bias+ReLU, 1x1 256->1024 +bias +residual(block input)
+ReLU, each a fused `tracea_conv2d` call on channels-last tensors resident in HBM. Inputs are
seeded synthetic tensors of the benchmark's shapes and distributions (|N(0,1)| activations,
Kaiming-normal weights, N(0,0.05) folded-BN bias); no dataset or checkpoint is involved.
The batch is sharded by image across GPUs with no collective on the data path (weak scaling:
256 images per GPU); torch.distributed only provides the start/stop barrier and the max over ranks.

One JSON line is printed by rank 0. `value` is TFLOP/s over all GPUs with the reference's FLOP
convention 2*M*K_out*(C*R*S) (src/optimizer/benchmark.rs:458-469). `e2e` is the same metric through
the C ABI with HOST (pinned) tensors, i.e. with the host<->device copies inside the timed region.
`roofline` is for the dominant kernel, the 3x3 conv. `cpu_baseline` times the CPU restatement of the
reference's SIMD conv path on the host cores (N=1 GPU runs only). `--impl reference` times only that.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BATCH_PER_GPU = 256
L2_BYTES = 126 * 1024 * 1024
WORKLOAD = ("resnet50_stage3_bottleneck_bf16: 1x1 1024->256 +bias+relu, 3x3 256->256 p1 +bias+relu, "
            "1x1 256->1024 +bias+residual+relu @14x14, %d images per GPU" % BATCH_PER_GPU)
# dram__bytes_read.sum + dram__bytes_write.sum of one 3x3-conv launch at N=256, from the ncu capture
# summarised in profiles/conv3x3_c256_k256_n256_bf16.md (26.95 MB read + 0.02 MB written; the 25.7 MB
# output is still dirty in L2 when the launch ends, which is why this is below the algorithmic bytes).
CONV3X3_NCU_TRAFFIC_BYTES = 26967552


def load_peaks():
    """Measured roofline denominators written by the test driver; fallback: an earlier measurement."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) while a region runs."""

    def __init__(self, index, period_s=0.004):
        self.index, self.period, self.samples, self.reasons = index, period_s, [], set()
        self.max_mhz, self._stop, self._thread, self._nvml = None, threading.Event(), None, None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None

    def _names(self, mask):
        n = self._nvml
        table = [("sw_power_cap", "nvmlClocksThrottleReasonSwPowerCap"),
                 ("hw_slowdown", "nvmlClocksThrottleReasonHwSlowdown"),
                 ("hw_thermal_slowdown", "nvmlClocksThrottleReasonHwThermalSlowdown"),
                 ("sw_thermal_slowdown", "nvmlClocksThrottleReasonSwThermalSlowdown"),
                 ("hw_power_brake", "nvmlClocksThrottleReasonHwPowerBrakeSlowdown")]
        return [name for name, attr in table if mask & getattr(n, attr, 0)]

    def _run(self):
        n = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM))
                self.reasons.update(self._names(n.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)))
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def block_oracle_inputs(n_images, seed=0):
    import numpy as np
    rng = np.random.default_rng(seed)
    x = np.abs(rng.standard_normal((n_images, 14, 14, 1024), dtype=np.float32)).transpose(0, 3, 1, 2)
    ws = [(rng.standard_normal(s, dtype=np.float32) * (2.0 / (s[1] * s[2] * s[3])) ** 0.5)
          for s in ((256, 1024, 1, 1), (256, 256, 3, 3), (1024, 256, 1, 1))]
    bs = [rng.standard_normal(k, dtype=np.float32) * 0.05 for k in (256, 256, 1024)]
    return x, ws, bs


def cpu_block_step(oracle, x, ws, bs, threads):
    """One pass of the bottleneck block on the host cores: the im2col + packed AVX2/FMA GEMM
    restatement of the reference's CPU engine, fp32."""
    y1 = oracle.conv2d_gemm(x, ws[0], bs[0], None, 1, 0, 1, "relu", threads)
    y2 = oracle.conv2d_gemm(y1, ws[1], bs[1], None, 1, 1, 1, "relu", threads)
    return oracle.conv2d_gemm(y2, ws[2], bs[2], x, 1, 0, 1, "relu", threads)


def block_flops(n_images):
    from tracea_b200 import resnet50
    return sum(resnet50.conv_flops(s, n_images) for s in resnet50.stage3_bottleneck())


def time_cpu_baseline(n_images, steps, warmup, budget_s=None):
    from oracle import oracle
    threads = os.cpu_count() or 1
    x, ws, bs = block_oracle_inputs(n_images)
    for _ in range(warmup):
        cpu_block_step(oracle, x, ws, bs, threads)
    t0 = time.perf_counter()
    done = 0
    for _ in range(steps):
        cpu_block_step(oracle, x, ws, bs, threads)
        done += 1
        if budget_s is not None and time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    return block_flops(n_images) * done / dt / 1e12, dt / done * 1e3, threads, done


def run_reference(args):
    """The reference's CPU conv path (no CUDA anywhere): rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n_sample = 8
    warm = max(1, min(args.warmup, 3))
    tflops, ms, threads, done = time_cpu_baseline(n_sample, args.steps, warm, budget_s=150.0)
    line = {
        "impl": "reference", "metric": "conv2d_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": done, "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": "%d images per step (of 256)" % n_sample},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": "bottleneck block on %d images per step, fp32, im2col + packed AVX2/FMA GEMM "
                                   "restatement of the reference's CPU engine (the reference is Rust and cannot "
                                   "be built here)" % n_sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist
    from tracea_b200 import build, ffi, resnet50, runner, shard

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the library has no CPU compute path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ["NCCL_DEBUG"] = "WARN"   # keep NCCL's version banner off stdout: one JSON line only
        dist.init_process_group("nccl", device_id=dev)
    if rank == 0:
        build.build()
    if world > 1:
        dist.barrier()
    lib = ffi.load()
    steps, warmup = args.steps, max(args.warmup, 3)
    n = BATCH_PER_GPU
    a, b = shard.shard_range(n * world, rank, world)     # this rank's images of the global batch
    assert b - a == n
    specs = resnet50.stage3_bottleneck()
    flops_step_rank = sum(resnet50.conv_flops(s, n) for s in specs)

    # Rotating buffer sets: one step touches ~257 MB (> L2) and the same set only comes back after
    # two other sets have passed through, so no step finds its inputs in L2.
    n_sets = 3
    torch.manual_seed(1234 + rank)
    stacks = []
    for i in range(n_sets):
        x = torch.randn((n, 1024, 14, 14), device=dev).abs_().to(torch.bfloat16).contiguous(
            memory_format=torch.channels_last)
        stacks.append(runner.ConvStack(specs, n, "bf16", dev, seed=7, inputs={"input": x}))
    set_bytes = sum(t.numel() * t.element_size() for t in stacks[0].tensors.values())
    stream = torch.cuda.current_stream(dev)

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    if args.only_layer is not None:
        # profiling aid: launch one layer of the block a few times and exit (no JSON line)
        j = [sp.name.split(".")[-1] for sp in specs].index(args.only_layer)
        for i in range(warmup + steps):
            stacks[i % n_sets].launch_one(j)
        barrier()
        print("launched %s %d times" % (specs[j].name, warmup + steps), flush=True)
        return

    for i in range(warmup):
        stacks[i % n_sets].forward()
    barrier()

    # ---- timed region: K steps, device-timed; an event between launches gives per-layer durations
    nl = len(specs)
    events = [torch.cuda.Event(enable_timing=True) for _ in range(steps * nl + 1)]
    launches_before = lib.tracea_b200_launch_count()
    with ClockSampler(local_rank) as clocks:
        events[0].record(stream)
        for i in range(steps):
            st = stacks[i % n_sets]
            for j in range(nl):
                st.launch_one(j)
                events[i * nl + j + 1].record(stream)
        barrier()
    launches = lib.tracea_b200_launch_count() - launches_before   # counted by the library itself, this rank
    status = lib.tracea_b200_device_status(local_rank)
    if status != 0:
        raise RuntimeError("a conv kernel gave up a bounded wait (device status %d)" % status)
    elapsed_ms = events[0].elapsed_time(events[-1])
    layer_ms = [0.0] * nl
    for i in range(steps):
        for j in range(nl):
            layer_ms[j] += events[i * nl + j].elapsed_time(events[i * nl + j + 1])
    layer_ms = [t / steps for t in layer_ms]
    elapsed_max = shard.max_over_ranks(elapsed_ms)
    ms_per_step = elapsed_max / steps
    value = flops_step_rank * world * steps / (elapsed_max * 1e-3) / 1e12

    # ---- end to end through the C ABI with host tensors (H2D + D2H inside the timed region)
    e2e_steps = max(3, min(steps, 15))
    host = {}
    g = torch.Generator().manual_seed(99 + rank)
    host["input"] = torch.randn((n, 1024, 14, 14), generator=g).abs_().to(torch.bfloat16).contiguous(
        memory_format=torch.channels_last).pin_memory()
    hw = {s.name: stacks[0].weights[s.name].cpu().contiguous(memory_format=torch.channels_last).pin_memory()
          for s in specs}
    hb = {s.name: stacks[0].biases[s.name].cpu().pin_memory() for s in specs}
    for s in specs:
        host[s.dst] = torch.empty((n, s.K, 14, 14), dtype=torch.bfloat16).contiguous(
            memory_format=torch.channels_last).pin_memory()
    from tracea_b200 import ops
    h2d = d2h = 0
    calls = []
    for s in specs:
        res = host[s.res] if s.res is not None else None
        kind = ops.parse_epilogue(s.epilogue, hb[s.name], res)
        calls.append((host[s.src], hw[s.name], hb[s.name], res, host[s.dst], s, kind))
        h2d += sum(t.numel() * t.element_size() for t in (host[s.src], hw[s.name], hb[s.name]))
        h2d += res.numel() * res.element_size() if res is not None else 0
        d2h += host[s.dst].numel() * host[s.dst].element_size()

    def e2e_step():
        for x_, w_, b_, r_, o_, s, kind in calls:
            ops.conv2d_into(x_, w_, o_, b_, r_, s.stride, s.pad, 1, 1, kind, stream=stream.cuda_stream)

    e2e_step()
    barrier()
    # every host-tensor call returns synchronised, so each step is timed on its own; the median is
    # reported because the PCIe root and host memory are shared with other tenants of the machine
    step_ms = []
    for _ in range(e2e_steps):
        t0 = time.perf_counter()
        e2e_step()
        torch.cuda.synchronize(dev)
        step_ms.append((time.perf_counter() - t0) * 1e3)
    barrier()
    step_ms.sort()
    e2e_median = shard.max_over_ranks(step_ms[len(step_ms) // 2])
    e2e_mean = shard.max_over_ranks(sum(step_ms) / len(step_ms))
    e2e_value = flops_step_rank * world / (e2e_median * 1e-3) / 1e12

    # ---- the whole ResNet-50 conv stack (53 fused convs), images/s, as an extra figure
    extra = {}
    if not args.no_resnet:
        try:
            nb = max(1, args.resnet_batch // world)   # config 5 shards a fixed global batch (strong scaling)
            rs = resnet50.resnet50_convs()
            img = torch.zeros((nb, 8, 224, 224), device=dev, dtype=torch.bfloat16).contiguous(
                memory_format=torch.channels_last)
            img[:, :3] = torch.randn((nb, 3, 224, 224), device=dev).to(torch.bfloat16)
            pooled = torch.randn((nb, 64, 56, 56), device=dev).abs_().to(torch.bfloat16).contiguous(
                memory_format=torch.channels_last)
            net = runner.ConvStack(rs, nb, "bf16", dev, seed=11, inputs={"image": img, "pooled": pooled})
            for _ in range(3):
                net.forward()
            barrier()
            # 53 launches per pass: replay them from a CUDA graph when capture works, else launch eagerly
            launch_mode = "eager"
            run_pass = net.forward
            if not args.no_graph:
                try:
                    net.capture()
                    run_pass, launch_mode = net.replay, "cuda-graph"
                except Exception:
                    torch.cuda.synchronize(dev)
            for _ in range(2):
                run_pass()
            barrier()
            r_steps = 10
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(r_steps):
                run_pass()
            e1.record(stream)
            barrier()
            r_ms = shard.max_over_ranks(e0.elapsed_time(e1)) / r_steps
            r_flops = sum(resnet50.conv_flops(s, nb) for s in rs)
            r_bytes = sum(resnet50.conv_bytes(s, nb) for s in rs)
            extra = {"workload": "ResNet-50 conv stack, 53 fused convs, bf16, global batch %d sharded over %d GPU(s)"
                                 % (nb * world, world), "scaling": "strong",
                     "images_per_s": nb * world / (r_ms * 1e-3), "ms_per_forward": r_ms,
                     "tflops": r_flops * world / (r_ms * 1e-3) / 1e12,
                     "algorithmic_gbs_per_gpu": r_bytes / (r_ms * 1e-3) / 1e9, "launches_per_forward": len(rs),
                     "launch_mode": launch_mode}
            del net, img, pooled
        except Exception as e:  # the extra figure must never take the headline line down
            extra = {"error": "%s: %s" % (type(e).__name__, e)}

    # ---- the operators either side of the conv path (GEMM, ConvTranspose2d), rank 0's GPU only, extra figures
    next_ops = {}
    if rank == 0 and not args.no_next_ops:
        try:
            next_ops = time_next_ops(dev, stream, lib, args.library_compare)
        except Exception as e:
            next_ops = {"error": "%s: %s" % (type(e).__name__, e)}
    barrier()

    if rank == 0:
        peaks = load_peaks()
        total_s = elapsed_max * 1e-3
        sustained = total_s >= 2.0
        peak_tf = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
        c2 = specs[1]
        c2_flops = resnet50.conv_flops(c2, n)
        achieved = c2_flops / (layer_ms[1] * 1e-3) / 1e12
        line = {
            "metric": "conv2d_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "batch_per_gpu": n, "global_batch": n * world,
                       "parallelism": "batch-sharded x%d, no collective" % world,
                       "l2": "%d rotating buffer sets of %.0f MB each (L2 is %.0f MB)" % (
                           n_sets, set_bytes / 1e6, L2_BYTES / 1e6)},
            "images_per_s": n * world / (ms_per_step * 1e-3),
            "layers": [{"name": s.name, "ms": layer_ms[j], "tflops": resnet50.conv_flops(s, n) / layer_ms[j] / 1e9,
                        "algorithmic_gbs": resnet50.conv_bytes(s, n) / layer_ms[j] / 1e6}
                       for j, s in enumerate(specs)],
            "roofline": {"kernel": "conv2d_igemm_sm100_kernel<bf16,256,pair> on the 3x3 256->256 conv", "bound": "tensor",
                         "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf,
                         "peak_source": "%s %s cuBLAS bf16" % (peaks["source"], "sustained" if sustained else "burst"),
                         "traffic": CONV3X3_NCU_TRAFFIC_BYTES, "algorithmic_bytes": resnet50.conv_bytes(c2, n),
                         "hbm_peak_gbs": peaks["hbm_gbs"]},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d * world,
                    "d2h_bytes_per_step": d2h * world, "steps": e2e_steps, "ms_per_step": e2e_median,
                    "ms_per_step_mean": e2e_mean, "stat": "median of the per-step times"},
            "gpu_launches": launches * world,
            "gpu_launches_per_step": launches / steps,
            "clocks": clocks.summary(),
            "resnet50": extra,
            "next_ops": next_ops,
        }
        if world == 1 and not args.no_cpu_baseline:
            tf, ms, threads, done = time_cpu_baseline(8, 1000, 1, budget_s=12.0)
            line["cpu_baseline"] = {
                "value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                "sample": "bottleneck block on 8 of the 256 images, fp32, %d passes (%.0f ms each): im2col + packed "
                          "AVX2/FMA GEMM restatement of the reference's CPU engine" % (done, ms)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def time_next_ops(dev, stream, lib, library_compare=False):
    """GEMM and ConvTranspose2d through tracea_gemm / tracea_conv_transpose2d on device tensors: 5 warm-up calls,
    then 20 timed calls between two CUDA events. Operand sets are larger than L2 (GEMM: 3 x 134 MB; the transposed
    convolution: 67 MB in, 134 MB out). FLOPs: 2*M*N*K; for the transposed convolution 2 * input pixels * C * K * R * S
    (every input pixel meets every tap once)."""
    import torch
    from tracea_b200 import ffi, ops

    def timed(fn, iters=20, warm=5):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        before = lib.tracea_b200_launch_count()
        e0.record(stream)
        for _ in range(iters):
            fn()
        e1.record(stream)
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / iters, (lib.tracea_b200_launch_count() - before) // iters

    out = {}
    g = torch.Generator(device=dev).manual_seed(5)
    M = K = N = 8192
    a = torch.randn((M, K), device=dev, dtype=torch.bfloat16, generator=g)
    bt = torch.randn((N, K), device=dev, dtype=torch.bfloat16, generator=g)       # [N][K] memory = b (K, N), strides (1, K)
    c = torch.empty((M, N), device=dev, dtype=torch.bfloat16)
    va, vb, vc = ops._view(a), ops._view(bt.t()), ops._view(c)
    ms, launches = timed(lambda: ffi.gemm_raw(va, vb, None, None, vc, ffi.EPILOGUE_IDENTITY, stream.cuda_stream))
    peaks = load_peaks()
    tf = 2.0 * M * N * K / (ms * 1e-3) / 1e12
    out["gemm"] = {"workload": "bf16 8192 x 8192 x 8192, b read in place as [N][K]", "ms": ms, "tflops": tf,
                   "launches_per_call": launches, "frac_of_measured_bf16_peak": tf / peaks["bf16_tflops"]}
    if library_compare:
        ms_lib, _ = timed(lambda: torch.matmul(a, bt.t(), out=c))
        out["gemm"]["cublas_tflops"] = 2.0 * M * N * K / (ms_lib * 1e-3) / 1e12
    del a, bt, c

    n, h, w, cin, kout, r, st, pad = 128, 32, 32, 256, 128, 4, 2, 1
    x = torch.randn((n, h, w, cin), device=dev, dtype=torch.bfloat16, generator=g)
    wt = torch.randn((kout, r, r, cin), device=dev, dtype=torch.bfloat16, generator=g) * (cin * r * r) ** -0.5
    ho = (h - 1) * st - 2 * pad + r
    y = torch.empty((n, ho, ho, kout), device=dev, dtype=torch.bfloat16)
    vx, vw, vy = ops._view(x), ops._view(wt), ops._view(y)
    ms, launches = timed(lambda: ffi.conv_transpose2d_raw(vx, vw, None, None, vy, (st, st), (pad, pad), (0, 0), (1, 1), 1,
                                                          ffi.EPILOGUE_IDENTITY, stream.cuda_stream))
    flops = 2.0 * n * h * w * cin * kout * r * r
    out["conv_transpose2d"] = {"workload": "bf16 x[128,32,32,256] * w[128,4,4,256], stride 2, pad 1 -> [128,64,64,128]",
                               "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12, "launches_per_call": launches}
    if library_compare:
        xc, wc = x.permute(0, 3, 1, 2), wt.permute(3, 0, 1, 2).contiguous(memory_format=torch.channels_last)
        ms_lib, _ = timed(lambda: torch.nn.functional.conv_transpose2d(xc, wc, None, st, pad))
        out["conv_transpose2d"]["cudnn_tflops"] = flops / (ms_lib * 1e-3) / 1e12
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-resnet", action="store_true", help="skip the ResNet-50 conv-stack extra figure")
    ap.add_argument("--resnet-batch", type=int, default=512, help="global batch of the conv-stack figure")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-next-ops", action="store_true", help="skip the GEMM / ConvTranspose2d extra figures")
    ap.add_argument("--library-compare", action="store_true",
                    help="also time torch.matmul / torch conv_transpose2d (cuBLAS / cuDNN) on the same shapes, for context")
    ap.add_argument("--no-graph", action="store_true", help="launch the conv stack eagerly instead of from a CUDA graph")
    ap.add_argument("--only-layer", choices=["c1", "c2", "c3"], default=None,
                    help="profiling aid: only launch this layer of the block, print no JSON")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

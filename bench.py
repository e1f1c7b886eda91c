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
the C ABI with HOST (pinned) tensors, one tracea_conv2d call per layer, i.e. with every tensor of every
call crossing the bus inside the timed region; `e2e_graph` runs the same block as a fused graph from
host memory (input copied in once, intermediates stay on the device, one output copied back).
`roofline` is for the dominant kernel, the 3x3 conv. `configs` times the other benchmark configurations
(one fp32 NCHW call, the fp16 README shape, the strided bf16 downsample, the reference's own 3x3 64->64
layer at its batch sizes), `resnet50` the 53-conv stack with a table per layer shape. `cpu_baseline`
times the reference's CPU conv path on the host cores (N=1 GPU runs only): what its Python op executes
on CPU tensors (torch.nn.functional.conv2d, tracea-python/src/conv2d.rs:80-136), next to the CPU
restatement of its SIMD GEMM engine fed by im2col and the scalar loop. `--impl reference` times only those.
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
# dram__bytes_read.sum + dram__bytes_write.sum of one 3x3-conv launch at N=256: NOT measured by this run but taken
# from the ncu capture summarised in profiles/conv3x3_c256_k256_n256_bf16.md (26.95 MB read + 0.02 MB written; the
# 25.7 MB output is still dirty in L2 when the launch ends, which is why this is below the algorithmic bytes).
CONV3X3_NCU_TRAFFIC_BYTES = 26967552
CONV3X3_NCU_TRAFFIC_SOURCE = "static: one ncu capture of this kernel at 256 images, profiles/conv3x3_c256_k256_n256_bf16.md"


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
    """B2: the oracle's im2col + packed AVX2/FMA GEMM path (restatement of src/kernels/cpu/gemm.rs), all cores."""
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


def time_cpu_torch(n_images, steps, warmup, budget_s=None):
    """B1: what the reference's conv op executes on CPU tensors -- torch.nn.functional.conv2d in fp32
    (tracea-python/src/conv2d.rs:80-136 falls back to it; its dtype guard forces fp32), bias / residual / ReLU as
    separate torch ops, all cores."""
    import torch
    import torch.nn.functional as F
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    x, ws, bs = block_oracle_inputs(n_images)
    tx = torch.from_numpy(x.copy()).contiguous(memory_format=torch.channels_last)
    tws = [torch.from_numpy(w).contiguous(memory_format=torch.channels_last) for w in ws]
    tbs = [torch.from_numpy(b) for b in bs]

    def step():
        with torch.no_grad():
            y1 = F.relu(F.conv2d(tx, tws[0], tbs[0]))
            y2 = F.relu(F.conv2d(y1, tws[1], tbs[1], 1, 1))
            return F.relu(F.conv2d(y2, tws[2], tbs[2]) + tx)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    done = 0
    for _ in range(steps):
        step()
        done += 1
        if budget_s is not None and time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    return block_flops(n_images) * done / dt / 1e12, dt / done * 1e3, threads, done


def time_cpu_scalar_config1(budget_s=4.0):
    """B0: the scalar restatement of cpu_conv2d (examples/verify_conv2d.rs:8-44) on benchmark configuration 1
    (fp32 x[1,64,56,56] * w[64,64,3,3] + bias, ReLU), one thread."""
    import numpy as np
    from oracle import oracle
    rng = np.random.default_rng(0)
    x = rng.uniform(-1, 1, (1, 64, 56, 56)).astype(np.float32)
    w = rng.uniform(-1, 1, (64, 64, 3, 3)).astype(np.float32)
    b = (rng.standard_normal(64) * 0.1).astype(np.float32)
    oracle.conv2d(x, w, b, None, 1, 1, 1, "relu")
    t0 = time.perf_counter()
    done = 0
    while done < 20 and time.perf_counter() - t0 < budget_s:
        oracle.conv2d(x, w, b, None, 1, 1, 1, "relu")
        done += 1
    dt = (time.perf_counter() - t0) / done
    return 2.0 * 56 * 56 * 64 * 64 * 9 / dt / 1e12, dt * 1e3, done


def cpu_baselines(n_images, budget_s):
    """The three CPU baselines of the reference's conv path, each on a bounded sample. The headline one is B1: it
    is literally the code the reference runs for this op on CPU tensors."""
    tf1, ms1, threads, done1 = time_cpu_torch(n_images, 1000, 1, budget_s=budget_s)
    tf2, ms2, _, done2 = time_cpu_baseline(n_images, 1000, 1, budget_s=budget_s)
    tf0, ms0, done0 = time_cpu_scalar_config1()
    main = {"value": tf1, "unit": "TFLOP/s", "cores": threads, "kind": "reference",
            "sample": "bottleneck block on %d of the 256 images, fp32, %d passes (%.0f ms each): "
                      "torch.nn.functional.conv2d on CPU tensors, the call the reference's conv op makes on CPU "
                      "(tracea-python/src/conv2d.rs:80-136)" % (n_images, done1, ms1)}
    others = {
        "simd_gemm_port": {"value": tf2, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                           "sample": "same block and sample, %d passes (%.0f ms each): im2col + packed AVX2/FMA GEMM "
                                     "restatement of the reference's CPU engine (src/kernels/cpu/gemm.rs)" % (done2, ms2)},
        "scalar_config1": {"value": tf0, "unit": "TFLOP/s", "cores": 1, "kind": "port",
                           "sample": "benchmark configuration 1 (fp32 x[1,64,56,56], 3x3 64->64, bias+ReLU), %d passes "
                                     "(%.0f ms each): scalar restatement of examples/verify_conv2d.rs:8-44" % (done0, ms0)},
    }
    return main, others


def run_reference(args):
    """The reference's CPU conv path (no CUDA anywhere): rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n_sample = 8
    warm = max(1, min(args.warmup, 3))
    tflops, ms, threads, done = time_cpu_torch(n_sample, args.steps, warm, budget_s=100.0)
    tf2, ms2, _, done2 = time_cpu_baseline(n_sample, args.steps, warm, budget_s=40.0)
    line = {
        "impl": "reference", "metric": "conv2d_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": done, "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": "%d images per step (of 256)" % n_sample},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "reference",
                         "sample": "bottleneck block on %d images per step, fp32: torch.nn.functional.conv2d on CPU "
                                   "tensors, the call the reference's conv op makes on CPU (tracea-python/src/conv2d.rs:"
                                   "80-136; the reference's Rust kernels cannot be built here and it has no CPU conv "
                                   "kernel of its own)" % n_sample},
        "cpu_baseline_simd_gemm_port": {"value": tf2, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                        "sample": "same block, %d passes of %.0f ms: im2col + packed AVX2/FMA GEMM "
                                                  "restatement of src/kernels/cpu/gemm.rs" % (done2, ms2)},
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
    # stdout carries exactly one JSON line: whatever libraries write to file descriptor 1 meanwhile (NCCL's version
    # banner and, when NCCL_DEBUG asks for them, its log lines) is sent to stderr, where it stays readable
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the library has no CPU compute path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
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

    for i in range(warmup):
        stacks[i % n_sets].forward()
    barrier()

    # ---- timed region: exactly K steps back to back, one event before and one after (consecutive launches overlap
    # their prologues with the previous kernel's tail: programmatic dependent launch, which any event in between
    # would switch off)
    nl = len(specs)
    e_begin, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches_before = lib.tracea_b200_launch_count()
    with ClockSampler(local_rank) as clocks:
        e_begin.record(stream)
        for i in range(steps):
            stacks[i % n_sets].forward()
        e_end.record(stream)
        barrier()
    launches = lib.tracea_b200_launch_count() - launches_before   # counted by the library itself, this rank
    status = lib.tracea_b200_device_status(local_rank)
    if status != 0:
        raise RuntimeError("a conv kernel gave up a bounded wait (device status %d)" % status)
    elapsed_ms = e_begin.elapsed_time(e_end)
    elapsed_max = shard.max_over_ranks(elapsed_ms)
    ms_per_step = elapsed_max / steps
    value = flops_step_rank * world * steps / (elapsed_max * 1e-3) / 1e12

    # ---- the same K steps once more with an event after every launch: per-layer durations (each launch now starts
    # only when the one before it has fully drained, so the three add up to slightly more than a step above)
    events = [torch.cuda.Event(enable_timing=True) for _ in range(steps * nl + 1)]
    events[0].record(stream)
    for i in range(steps):
        st = stacks[i % n_sets]
        for j in range(nl):
            st.launch_one(j)
            events[i * nl + j + 1].record(stream)
    barrier()
    layer_ms = [0.0] * nl
    for i in range(steps):
        for j in range(nl):
            layer_ms[j] += events[i * nl + j].elapsed_time(events[i * nl + j + 1])
    layer_ms = [t / steps for t in layer_ms]

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

    # ---- the same block as a fused graph from host memory: input H2D once, chain on device, output D2H once
    e2e_graph = {}
    try:
        e2e_graph = time_e2e_graph(dev, n, stacks[0], specs, host["input"], flops_step_rank, world, e2e_steps, barrier, shard)
    except Exception as e:
        e2e_graph = {"error": "%s: %s" % (type(e).__name__, e)}

    # ---- the whole ResNet-50 conv stack (53 fused convs), images/s, as an extra figure
    extra = {}
    if not args.no_resnet:
        try:
            nb = max(1, args.resnet_batch // world)   # config 5 shards a fixed global batch (strong scaling)
            rs = resnet50.resnet50_convs()
            img = torch.randn((nb, 3, 224, 224), device=dev).to(torch.bfloat16).contiguous(
                memory_format=torch.channels_last)      # a true 3-channel NHWC image
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
            extra["layers"] = stack_layer_table(net, rs, nb, load_peaks(), stream)
            del net, img, pooled
        except Exception as e:  # the extra figure must never take the headline line down
            extra = {"error": "%s: %s" % (type(e).__name__, e)}

    # ---- the other benchmark configurations and the reference's own layer, rank 0's GPU only
    configs = {}
    if rank == 0 and not args.no_configs:
        try:
            configs = time_configs(dev, stream, lib, load_peaks())
        except Exception as e:
            configs = {"error": "%s: %s" % (type(e).__name__, e)}
    barrier()

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
            "layers_note": "per-layer times come from a second pass of the same steps with a CUDA event after every "
                           "launch; the headline pass has none, so that consecutive launches overlap (programmatic "
                           "dependent launch)",
            "layers": [{"name": s.name, "ms": layer_ms[j], "tflops": resnet50.conv_flops(s, n) / layer_ms[j] / 1e9,
                        "algorithmic_gbs": resnet50.conv_bytes(s, n) / layer_ms[j] / 1e6}
                       for j, s in enumerate(specs)],
            "roofline": {"kernel": "conv2d_igemm_sm100_kernel<bf16,256,pair> on the 3x3 256->256 conv", "bound": "tensor",
                         "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf,
                         "peak_source": "%s %s cuBLAS bf16" % (peaks["source"], "sustained" if sustained else "burst"),
                         "traffic": CONV3X3_NCU_TRAFFIC_BYTES, "traffic_source": CONV3X3_NCU_TRAFFIC_SOURCE,
                         "algorithmic_bytes": resnet50.conv_bytes(c2, n),
                         "hbm_peak_gbs": peaks["hbm_gbs"]},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d * world,
                    "d2h_bytes_per_step": d2h * world, "steps": e2e_steps, "ms_per_step": e2e_median,
                    "ms_per_step_mean": e2e_mean, "stat": "median of the per-step times",
                    "what": "three tracea_conv2d calls on pinned host tensors: every tensor of every call crosses the bus",
                    "bus_gbs_per_rank": (h2d + d2h) / (e2e_median * 1e-3) / 1e9},
            "e2e_graph": e2e_graph,
            "gpu_launches": launches * world,
            "gpu_launches_per_step": launches / steps,
            "clocks": clocks.summary(),
            "configs": configs,
            "resnet50": extra,
            "next_ops": next_ops,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"], line["cpu_baselines_other"] = cpu_baselines(8, budget_s=8.0)
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def time_e2e_graph(dev, n, stack, specs, host_in, flops_step_rank, world, steps, barrier, shard):
    """The bottleneck block as a GraphTopology (conv-bn-relu x2, conv-bn-add-relu), fused to three convs with the
    BatchNorms folded, run from pinned HOST memory through GraphRunner.run_host: the timed region holds the copy of
    the input to the device, the three kernels per image chunk and the copy of the output back."""
    import torch
    from tracea_b200 import graph as G
    g = G.bottleneck_graph(n, 1024, 256, 14)
    params = {}
    for o in g["operators"]:
        oid, name = G.op_id(o), G.op_body(o)["name"]
        if G.op_kind(o) != "Input" or oid == 0:
            continue
        bn = int(name.split(".")[0])
        c = 1024 if bn == 8 else 256
        bias = stack.biases[specs[{2: 0, 5: 1, 8: 2}[bn]].name].cpu()
        params[oid] = {"gamma": torch.ones(c), "beta": bias, "mean": torch.zeros(c), "var": torch.ones(c)}[name.split(".")[1]]
    for conv_id, sp in zip((1, 4, 7), specs):
        params[conv_id] = {"weight": stack.weights[sp.name].float().cpu()}
    runner_ = G.GraphRunner(G.fuse(g), params, dtype=torch.bfloat16)
    host_out = torch.empty((n, 1024, 14, 14), dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last).pin_memory()
    runner_.run_host({0: host_in}, {7: host_out}, device=dev, chunks=8)
    barrier()
    ms = []
    for _ in range(steps):
        t0 = time.perf_counter()
        runner_.run_host({0: host_in}, {7: host_out}, device=dev, chunks=8)
        ms.append((time.perf_counter() - t0) * 1e3)
    barrier()
    ms.sort()
    med = shard.max_over_ranks(ms[len(ms) // 2])
    h2d = host_in.numel() * host_in.element_size()
    d2h = host_out.numel() * host_out.element_size()
    return {"value": flops_step_rank * world / (med * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": med,
            "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world, "steps": steps,
            "bus_gbs_per_rank": (h2d + d2h) / (med * 1e-3) / 1e9,
            "what": "fused graph from pinned host memory (GraphRunner.run_host): input in, three convs per image chunk on "
                    "the device, output out; copy-in, kernels and copy-out of different chunks overlap"}


def stack_layer_table(net, rs, nb, peaks, stream):
    """One row per distinct layer shape of the conv stack: launches, time (min of 3 eager passes, an event
    between launches), roofline bound max(FLOPs / bf16 peak, algorithmic bytes / HBM bandwidth) and their ratio."""
    import torch
    from tracea_b200 import resnet50
    reps = 3
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(rs) + 1)] for _ in range(reps)]
    for r in range(reps):
        ev[r][0].record(stream)
        for j in range(len(rs)):
            net.launch_one(j)
            ev[r][j + 1].record(stream)
    torch.cuda.synchronize()
    rows = {}
    for j, s in enumerate(rs):
        ms = min(ev[r][j].elapsed_time(ev[r][j + 1]) for r in range(reps))
        fl, by = resnet50.conv_flops(s, nb), resnet50.conv_bytes(s, nb)
        bound = max(fl / (peaks["bf16_tflops"] * 1e12), by / (peaks["hbm_gbs"] * 1e9)) * 1e3
        key = "C%d H%d K%d %dx%d/%d %s" % (s.C, s.H, s.K, s.R, s.S, s.stride, s.epilogue)
        row = rows.setdefault(key, {"shape": key, "count": 0, "ms": 0.0, "bound_ms": 0.0, "gflop": 0.0, "mbytes": 0.0})
        row["count"] += 1
        row["ms"] += ms
        row["bound_ms"] += bound
        row["gflop"] += fl / 1e9
        row["mbytes"] += by / 1e6
    out = []
    for row in rows.values():
        row["bound"] = "tensor" if row["gflop"] / peaks["bf16_tflops"] > row["mbytes"] / peaks["hbm_gbs"] else "hbm"
        row["ratio_to_bound"] = row["ms"] / row["bound_ms"]
        for k in ("ms", "bound_ms", "gflop", "mbytes", "ratio_to_bound"):
            row[k] = round(row[k], 4)
        out.append(row)
    out.sort(key=lambda r: -(r["ms"] - r["bound_ms"]))
    return out


def time_configs(dev, stream, lib, peaks):
    """The benchmark configurations that are not the headline block, each through tracea_conv2d on device tensors
    laid out as the configuration states them (configuration 1 and 2: NCHW activations and OIHW weights, so the
    layout adapters run inside every call and are part of the time), plus the reference's own benchmark layer
    (3x3 64->64 at 56x56, examples/resnet_bench.rs:28-47) at its batch sizes. Device time: CUDA events around
    `iters` back-to-back calls over rotating operand sets; host time: wall clock per call of issuing them (the
    argument structs are built once outside the loop, so this is the C entry point's own cost plus the ctypes call)."""
    import ctypes
    import torch
    from tracea_b200 import ffi, ops
    dt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}

    def one(name, n, c, h, k, r, stride, pad, dtype, epilogue, nchw, iters, sets=3, peak_tf=None):
        g = torch.Generator(device=dev).manual_seed(3)
        cl = (lambda t: t.contiguous()) if nchw else (lambda t: t.contiguous(memory_format=torch.channels_last))
        ho = (h + 2 * pad - r) // stride + 1
        w = cl((torch.randn((k, c, r, r), device=dev, generator=g) * (2.0 / (c * r * r)) ** 0.5).to(dt[dtype]))
        bias = torch.randn((k,), device=dev, generator=g) * 0.1 if "bias" in epilogue else None
        kind = ops.parse_epilogue(epilogue or None, bias, None)
        xs = [cl(torch.randn((n, c, h, h), device=dev, generator=g).to(dt[dtype])) for _ in range(sets)]
        outs = [cl(torch.empty((n, k, ho, ho), device=dev, dtype=dt[dtype])) for _ in range(sets)]
        # arguments marshalled once, as a C caller of the ABI would hold them: the timed loop is the C entry point alone
        vw, vb = ops._view(w), (ops._view(bias) if bias is not None else None)
        views = [(ops._view(xs[i]), ops._view(outs[i])) for i in range(sets)]
        params = ffi.Conv2dParams(stride, stride, pad, pad, 1, 1, 1, int(kind), ctypes.c_void_p(stream.cuda_stream))

        def call(i):
            vx, vo = views[i % sets]
            st = lib.tracea_conv2d(vx.c, vw.c, ctypes.byref(vb.c) if vb is not None else None, None, ctypes.byref(vo.c),
                                   params)
            if st != ffi.SUCCESS:
                raise ffi.TraceaError(st, ffi.last_error())
        for i in range(5):
            call(i)
        torch.cuda.synchronize(dev)
        before = lib.tracea_b200_launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record(stream)
        for i in range(iters):
            call(i)
        e1.record(stream)
        host_us = (time.perf_counter() - t0) / iters * 1e6
        torch.cuda.synchronize(dev)
        us = e0.elapsed_time(e1) / iters * 1e3
        es = 4 if dtype == "f32" else 2
        flops = 2.0 * n * ho * ho * k * c * r * r
        nbytes = (n * c * h * h + k * c * r * r + n * k * ho * ho) * es + (k * 4 if bias is not None else 0)
        peak = peak_tf if peak_tf is not None else peaks["bf16_tflops"]
        bound_us = max(flops / (peak * 1e12), nbytes / (peaks["hbm_gbs"] * 1e9)) * 1e6
        return {"workload": name, "us_per_call": us, "host_us_per_call": host_us, "tflops": flops / us / 1e6,
                "algorithmic_gbs": nbytes / us / 1e3, "bound_us": bound_us, "frac_of_bound": bound_us / us,
                "launches_per_call": (lib.tracea_b200_launch_count() - before) // iters,
                "layout": "NCHW / OIHW as stated (adapters inside the call)" if nchw else "channels-last"}

    tf32_peak = peaks["bf16_tflops"] / 2.0   # TF32 runs at half the bf16 rate
    out = {
        "config1": one("fp32 (TF32) x[1,64,56,56] * w[64,64,3,3] s1 p1 +bias+relu", 1, 64, 56, 64, 3, 1, 1, "f32",
                       "bias+relu", True, 200, peak_tf=tf32_peak),
        "config2": one("fp16 x[1,64,224,224] * w[128,64,3,3] s1 p0", 1, 64, 224, 128, 3, 1, 0, "f16", "", True, 100),
        "config2_channels_last": one("fp16 x[1,64,224,224] * w[128,64,3,3] s1 p0, channels-last tensors", 1, 64, 224, 128, 3,
                                     1, 0, "f16", "", False, 100),
        "config4": one("bf16 x[256,128,56,56] * w[256,128,3,3] s2 p1 +bias+silu", 256, 128, 56, 256, 3, 2, 1, "bf16",
                       "bias+silu", False, 30),
    }
    for batch in (32, 64, 256):
        out["reference_layer_b%d" % batch] = one(
            "bf16 x[%d,64,56,56] * w[64,64,3,3] s1 p1 +bias+relu (the reference's benchmark layer)" % batch, batch, 64, 56,
            64, 3, 1, 1, "bf16", "bias+relu", False, 60 if batch < 256 else 30, sets=3 if batch < 256 else 3)
    out["note"] = ("bound_us = max(FLOPs / measured tensor peak, algorithmic bytes / measured HBM bandwidth); TF32 is "
                   "given half the bf16 peak; configurations 1 and 2 are single images: launch latency, not the roofline, "
                   "sets their time")
    return out


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
    ap.add_argument("--no-configs", action="store_true", help="skip the figures of the other benchmark configurations")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

"""Runs a chain of fused convolutions (a bottleneck block, the whole ResNet-50 conv stack) through
the C ABI with every tensor resident on one GPU.

This is the counterpart of the reference's per-layer benchmark object (`NVRTCConvBenchmark`,
src/optimizer/benchmark.rs:635-930: allocate, fill, warm up, launch) and of the launch-replay part
of its graph executor (src/runtime/executor/mod.rs:38-77), reduced to what the conv path needs:
buffers are allocated once, ctypes argument blocks are built once, and `forward()` only issues
`tracea_conv2d` calls on the current stream.
"""
import ctypes

import torch

from . import ffi, ops
from .resnet50 import out_hw

_TORCH_DT = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}


def _channels_last_empty(shape, dtype, device):
    return torch.empty(shape, dtype=dtype, device=device, memory_format=torch.channels_last)


class ConvStack:
    """specs: list of resnet50.ConvSpec. inputs: dict name -> logical-NCHW tensor (channels-last
    memory) for every tensor the specs read but do not produce. Weights are OIHW-shaped
    channels-last tensors (KRSC memory); biases fp32."""

    def __init__(self, specs, n_images, dtype="bf16", device="cuda", seed=0, inputs=None, weights=None):
        self.specs = list(specs)
        self.n = n_images
        self.dtype = _TORCH_DT[dtype]
        self.device = torch.device(device)
        self.tensors = dict(inputs or {})
        self.weights = {}
        self.biases = {}
        gen = torch.Generator(device="cpu").manual_seed(seed)
        for sp in self.specs:
            if weights is not None:
                w, b = weights[sp.name]
            else:
                fan_in = sp.C * sp.R * sp.S
                w = torch.randn((sp.K, sp.C, sp.R, sp.S), generator=gen) * (2.0 / fan_in) ** 0.5
                b = torch.randn((sp.K,), generator=gen) * 0.05
            # an input supplied with more channels than the layer reads (an RGB image stored with zero-padded
            # channels) gets weights padded to match; a true 3-channel image is taken as it is
            src = self.tensors.get(sp.src)
            c_phys = src.shape[1] if src is not None and src.shape[1] > sp.C else sp.C
            if c_phys != sp.C:
                wp = torch.zeros((sp.K, c_phys, sp.R, sp.S))
                wp[:, :sp.C] = w
                w = wp
            self.weights[sp.name] = w.to(self.dtype).to(self.device).contiguous(memory_format=torch.channels_last)
            self.biases[sp.name] = b.float().to(self.device)
        for sp in self.specs:
            if sp.src not in self.tensors:
                raise KeyError("input tensor %r was not supplied" % sp.src)
            ho, wo = out_hw(sp.H, sp.R, sp.stride, sp.pad), out_hw(sp.W, sp.S, sp.stride, sp.pad)
            self.tensors[sp.dst] = _channels_last_empty((n_images, sp.K, ho, wo), self.dtype, self.device)
        self._calls = [self._prepare(sp) for sp in self.specs]
        self._lib = ffi.load()

    def _prepare(self, sp):
        x = self.tensors[sp.src]
        w = self.weights[sp.name]
        if x.shape[1] != w.shape[1]:
            raise ValueError("%s: input has %d channels, weights expect %d" % (sp.name, x.shape[1], w.shape[1]))
        res = self.tensors[sp.res] if sp.res is not None else None
        bias = self.biases[sp.name]
        kind = ops.parse_epilogue(sp.epilogue, bias, res)
        views = (ops._view(x), ops._view(w), ops._view(bias), ops._view(res) if res is not None else None,
                 ops._view(self.tensors[sp.dst]))
        params = ffi.Conv2dParams(sp.stride, sp.stride, sp.pad, sp.pad, 1, 1, 1, int(kind), None)
        return sp, views, params

    def forward(self, stream=None):
        """Enqueue every conv of the chain, in order, on `stream` (default: torch's current stream)."""
        if stream is None:
            stream = torch.cuda.current_stream(self.device).cuda_stream
        lib = self._lib
        for sp, (vx, vw, vb, vr, vo), params in self._calls:
            params.stream = ctypes.c_void_p(stream)
            st = lib.tracea_conv2d(vx.c, vw.c, ctypes.byref(vb.c), ctypes.byref(vr.c) if vr is not None else None,
                                   ctypes.byref(vo.c), params)
            if st != ffi.SUCCESS:
                raise ffi.TraceaError(st, "%s: %s" % (sp.name, ffi.last_error()))
        return self.tensors[self.specs[-1].dst]

    def launch_one(self, index, stream=None):
        """Enqueue only conv number `index` (used to time a single layer between two events)."""
        if stream is None:
            stream = torch.cuda.current_stream(self.device).cuda_stream
        sp, (vx, vw, vb, vr, vo), params = self._calls[index]
        params.stream = ctypes.c_void_p(stream)
        st = self._lib.tracea_conv2d(vx.c, vw.c, ctypes.byref(vb.c), ctypes.byref(vr.c) if vr is not None else None,
                                     ctypes.byref(vo.c), params)
        if st != ffi.SUCCESS:
            raise ffi.TraceaError(st, "%s: %s" % (sp.name, ffi.last_error()))

    def capture(self):
        """Record one forward pass into a CUDA graph (launch-bound chains: 53 small launches cost more
        host time than GPU time at small batch). Returns the graph; `replay()` runs it. The pass is run
        once eagerly first so that every one-time set-up (kernel attributes, scratch pool growth) is
        done before capture."""
        self.forward()
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.forward()
        self._graph = graph
        return graph

    def replay(self):
        self._graph.replay()
        return self.tensors[self.specs[-1].dst]

    @property
    def num_launches(self):
        return len(self._calls)

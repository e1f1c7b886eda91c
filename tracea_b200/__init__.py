"""tracea_b200: a B200 (sm_100a) implicit-GEMM Conv2d behind Tracea's operator surface.

Layers, bottom up:
  csrc/            hand-written CUDA (TMA im2col -> tcgen05.mma -> TMEM -> fused epilogue) + the C ABI
  ffi              ctypes binding of that C ABI (include/tracea_b200.h)
  ops              the reference's Python operator surface (tracea.ops.conv2d, gemm, conv_transpose2d, Context.conv2d)
  nn               TraceaConv2d / patch_conv2d, the reference's torch.nn drop-in
  graph            GraphTopology JSON -> Conv+BN+Add+ReLU fusion -> fused conv graphs on the kernel

Importing the package does not load the compiled library; the first call does, and raises if the
library has not been built. There is no fallback implementation.
"""
from . import ffi  # noqa: F401

__version__ = "0.1.0"

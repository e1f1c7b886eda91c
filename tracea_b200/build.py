"""Ahead-of-time build of libtracea_b200.so (nvcc, sm_100a only). Cross-compiles without a GPU.

This replaces the reference's run-time path NVRTC -> PTX -> cuModuleLoadData
(src/runtime/manager/kernel.rs:123-327): there is no code generation at run time here.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libtracea_b200.so")
SOURCES = [os.path.join(CSRC, "tracea_ffi.cu")]
HEADERS = [os.path.join(CSRC, f) for f in ("conv2d_sm100.cuh", "conv2d_window_sm100.cuh", "conv2d_rowband_sm100.cuh", "ptx_sm100.cuh", "layout_kernels.cuh")] + [
    os.path.join(HERE, "..", "include", "tracea_b200.h")]

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared", "-cudart", "static",
]


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(p) > t for p in SOURCES + HEADERS)


def build(force=False, verbose=False):
    """Compile the library in-tree when it is missing or older than its sources."""
    if not force and not needs_build():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB] + SOURCES
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        sys.stderr.write(res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))

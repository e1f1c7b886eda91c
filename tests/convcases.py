"""Seeded inputs and comparison helpers shared by the parity tests.

Synthetic tensors stand in for the image batches and trained weights the benchmark configs name:
same shapes, dtypes and value distributions, drawn from a counter-based Philox stream keyed by
(seed, tensor tag) so that every test, rank and run regenerates identical data.
"""
import zlib

import numpy as np

TOL_16BIT = 1e-2   # max|out - ref| <= 1e-2 * max|ref| for fp16 / bf16 inputs with fp32 accumulation
TOL_TF32 = 5e-3    # max|out - ref| <= 5e-3 * max|ref| for fp32 inputs computed as TF32


def rng_for(seed, tag):
    return np.random.Generator(np.random.Philox(key=[seed, zlib.crc32(tag.encode()) & 0xFFFFFFFF]))


def uniform(shape, seed, tag, lo=-1.0, hi=1.0):
    return rng_for(seed, tag).uniform(lo, hi, size=shape).astype(np.float32)


def normal(shape, seed, tag, std=1.0):
    return (rng_for(seed, tag).standard_normal(size=shape) * std).astype(np.float32)


def kaiming(shape, seed, tag):
    """Kaiming-normal weights for an OIHW filter: std = sqrt(2 / fan_in)."""
    fan_in = shape[1] * shape[2] * shape[3]
    return normal(shape, seed, tag, (2.0 / fan_in) ** 0.5)


def round_to(a, dtype):
    """Round an fp32 array to the storage type `dtype` ('f32' | 'f16' | 'bf16') and back (RNE)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    if dtype == "f32":
        return a
    if dtype == "f16":
        return a.astype(np.float16).astype(np.float32)
    if dtype == "bf16":
        u = a.view(np.uint32).astype(np.uint64)
        u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
        return u.astype(np.uint32).view(np.float32).reshape(a.shape)
    raise ValueError(dtype)


def channels_last(a):
    """Logical NCHW view over dense NHWC memory."""
    return np.ascontiguousarray(a.transpose(0, 2, 3, 1)).transpose(0, 3, 1, 2)


def rel_err(out, ref):
    ref = np.asarray(ref, dtype=np.float64)
    out = np.asarray(out, dtype=np.float64)
    scale = max(float(np.abs(ref).max()), 1e-30)
    return float(np.abs(out - ref).max()) / scale


def tol_for(dtype):
    return TOL_TF32 if dtype == "f32" else TOL_16BIT

"""ctypes front end of oracle/conv2d_oracle.c (the CPU restatement of the reference's conv) and of
oracle/next_ops_oracle.c (ConvTranspose2d and GEMM with the same epilogue).

TEST INFRASTRUCTURE: only tests/, the smoke check and the benchmark's CPU-baseline leg import this
module. The tracea_b200 package never does.

All tensors are numpy float32 arrays in their *logical* index order (x: N,C,H,W; w: K,C,R,S;
out: N,K,Ho,Wo); the physical layout is whatever the array's strides say, so a channels-last array
(``np.transpose`` view of NHWC memory) is read in place.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None

ACT = {"none": 0, "relu": 1, "gelu": 2, "silu": 3}


class _Desc(ctypes.Structure):
    _fields_ = [
        ("N", ctypes.c_longlong), ("C", ctypes.c_longlong), ("H", ctypes.c_longlong), ("W", ctypes.c_longlong),
        ("K", ctypes.c_longlong), ("R", ctypes.c_longlong), ("S", ctypes.c_longlong),
        ("stride_h", ctypes.c_longlong), ("stride_w", ctypes.c_longlong),
        ("pad_h", ctypes.c_longlong), ("pad_w", ctypes.c_longlong),
        ("dil_h", ctypes.c_longlong), ("dil_w", ctypes.c_longlong),
        ("xs", ctypes.c_longlong * 4), ("ws", ctypes.c_longlong * 4),
        ("os", ctypes.c_longlong * 4), ("rs", ctypes.c_longlong * 4),
        ("act", ctypes.c_int), ("acc_double", ctypes.c_int),
    ]


class _ConvTDesc(ctypes.Structure):
    _fields_ = [
        ("N", ctypes.c_longlong), ("H", ctypes.c_longlong), ("W", ctypes.c_longlong), ("C", ctypes.c_longlong),
        ("K", ctypes.c_longlong), ("R", ctypes.c_longlong), ("S", ctypes.c_longlong),
        ("stride_h", ctypes.c_longlong), ("stride_w", ctypes.c_longlong),
        ("pad_h", ctypes.c_longlong), ("pad_w", ctypes.c_longlong),
        ("opad_h", ctypes.c_longlong), ("opad_w", ctypes.c_longlong),
        ("xs", ctypes.c_longlong * 4), ("ws", ctypes.c_longlong * 4),
        ("os", ctypes.c_longlong * 4), ("rs", ctypes.c_longlong * 4),
        ("act", ctypes.c_int),
    ]


class _GemmDesc(ctypes.Structure):
    _fields_ = [
        ("M", ctypes.c_longlong), ("N", ctypes.c_longlong), ("K", ctypes.c_longlong),
        ("as_", ctypes.c_longlong * 2), ("bs", ctypes.c_longlong * 2), ("cs", ctypes.c_longlong * 2),
        ("rs", ctypes.c_longlong * 2),
        ("act", ctypes.c_int),
    ]


def build(force=False):
    """Compile liboracle.so with gcc (needs nothing but libc, libm and libgomp)."""
    newest = max(os.path.getmtime(os.path.join(_HERE, f)) for f in ("conv2d_oracle.c", "next_ops_oracle.c", "Makefile"))
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < newest:
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        fp = ctypes.POINTER(ctypes.c_float)
        _lib.oracle_conv2d.argtypes = [ctypes.POINTER(_Desc), fp, fp, fp, fp, fp]
        _lib.oracle_conv2d.restype = ctypes.c_int
        _lib.oracle_conv2d_gemm.argtypes = [ctypes.POINTER(_Desc), fp, fp, fp, fp, fp, ctypes.c_int]
        _lib.oracle_conv2d_gemm.restype = ctypes.c_int
        _lib.oracle_conv2d_points.argtypes = [ctypes.POINTER(_Desc), fp, fp, fp, fp,
                                              ctypes.POINTER(ctypes.c_longlong), ctypes.c_longlong, fp]
        _lib.oracle_conv2d_points.restype = ctypes.c_int
        _lib.oracle_num_threads.restype = ctypes.c_int
        _lib.oracle_conv_transpose2d.argtypes = [ctypes.POINTER(_ConvTDesc), fp, fp, fp, fp, fp]
        _lib.oracle_conv_transpose2d.restype = ctypes.c_int
        _lib.oracle_gemm.argtypes = [ctypes.POINTER(_GemmDesc), fp, fp, fp, fp, fp]
        _lib.oracle_gemm.restype = ctypes.c_int
    return _lib


def _pair(v):
    return (int(v), int(v)) if np.isscalar(v) else (int(v[0]), int(v[1]))


def out_shape(xshape, wshape, stride=1, padding=0, dilation=1):
    sh, sw = _pair(stride)
    ph, pw = _pair(padding)
    dh, dw = _pair(dilation)
    N, _, H, W = xshape
    K, _, R, S = wshape
    Ho = (H + 2 * ph - dh * (R - 1) - 1) // sh + 1
    Wo = (W + 2 * pw - dw * (S - 1) - 1) // sw + 1
    return (N, K, Ho, Wo)


def _estrides(a):
    assert a.dtype == np.float32
    return [s // 4 for s in a.strides]


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def _desc(x, w, out, residual, stride, padding, dilation, act, acc_double):
    d = _Desc()
    d.N, d.C, d.H, d.W = x.shape
    d.K, cw, d.R, d.S = w.shape
    assert cw == d.C, "channel mismatch"
    d.stride_h, d.stride_w = _pair(stride)
    d.pad_h, d.pad_w = _pair(padding)
    d.dil_h, d.dil_w = _pair(dilation)
    d.xs = (ctypes.c_longlong * 4)(*_estrides(x))
    d.ws = (ctypes.c_longlong * 4)(*_estrides(w))
    if out is not None:
        d.os = (ctypes.c_longlong * 4)(*_estrides(out))
    if residual is not None:
        d.rs = (ctypes.c_longlong * 4)(*_estrides(residual))
    d.act = ACT[act]
    d.acc_double = int(acc_double)
    return d


def conv2d(x, w, bias=None, residual=None, stride=1, padding=0, dilation=1, act="none",
           acc_double=False, channels_last_out=False):
    """Scalar restatement of examples/verify_conv2d.rs:8-44 plus the fused epilogue. Returns an
    array of logical shape (N, K, Ho, Wo) (channels-last memory when ``channels_last_out``)."""
    shape = out_shape(x.shape, w.shape, stride, padding, dilation)
    if channels_last_out:
        out = np.empty((shape[0], shape[2], shape[3], shape[1]), np.float32).transpose(0, 3, 1, 2)
    else:
        out = np.empty(shape, np.float32)
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np.float32)
    d = _desc(x, w, out, residual, stride, padding, dilation, act, acc_double)
    rc = lib().oracle_conv2d(ctypes.byref(d), _ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out))
    assert rc == 0
    return out


def conv2d_gemm(x, w, bias=None, residual=None, stride=1, padding=0, dilation=1, act="none",
                threads=0, channels_last_out=True):
    """im2col + packed AVX2/FMA GEMM (restatement of src/kernels/cpu/gemm.rs). ``x`` must be a
    channels-last view (dense NHWC memory)."""
    shape = out_shape(x.shape, w.shape, stride, padding, dilation)
    if channels_last_out:
        out = np.empty((shape[0], shape[2], shape[3], shape[1]), np.float32).transpose(0, 3, 1, 2)
    else:
        out = np.empty(shape, np.float32)
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np.float32)
    d = _desc(x, w, out, residual, stride, padding, dilation, act, False)
    rc = lib().oracle_conv2d_gemm(ctypes.byref(d), _ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out),
                                  int(threads))
    if rc != 0:
        raise ValueError("oracle_conv2d_gemm: x must be dense NHWC memory (rc=%d)" % rc)
    return out


def conv2d_points(x, w, idx, bias=None, residual=None, stride=1, padding=0, dilation=1, act="none",
                  acc_double=True):
    """Values of selected output points; ``idx`` is an (n_points, 4) array of (n, k, ho, wo)."""
    idx = np.ascontiguousarray(idx, dtype=np.int64)
    vals = np.empty(idx.shape[0], np.float32)
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np.float32)
    d = _desc(x, w, None, residual, stride, padding, dilation, act, acc_double)
    rc = lib().oracle_conv2d_points(ctypes.byref(d), _ptr(x), _ptr(w), _ptr(bias), _ptr(residual),
                                    idx.ctypes.data_as(ctypes.POINTER(ctypes.c_longlong)), idx.shape[0],
                                    _ptr(vals))
    assert rc == 0
    return vals


def num_threads():
    return lib().oracle_num_threads()


def conv_transpose_out_shape(xshape, wshape, stride=1, padding=0, output_padding=0):
    """x (N, H, W, C), w (K, R, S, C) -> (N, Ho, Wo, K); Ho = (H-1)*stride - 2*pad + R + output_padding
    (src/interface/c_bindings.rs:343-344)."""
    sh, sw = _pair(stride)
    ph, pw = _pair(padding)
    oh, ow = _pair(output_padding)
    N, H, W, _ = xshape
    K, R, S, _ = wshape
    return (N, (H - 1) * sh - 2 * ph + R + oh, (W - 1) * sw - 2 * pw + S + ow, K)


def conv_transpose2d(x, w, bias=None, residual=None, stride=1, padding=0, output_padding=0, act="none"):
    """Scatter restatement of examples/verify_conv_transpose.rs:12-52 plus the fused epilogue.
    x (N, H, W, C), w (K, R, S, C), residual / result (N, Ho, Wo, K): float32 arrays of any strides."""
    shape = conv_transpose_out_shape(x.shape, w.shape, stride, padding, output_padding)
    out = np.empty(shape, np.float32)
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np.float32)
    d = _ConvTDesc()
    d.N, d.H, d.W, d.C = x.shape
    d.K, d.R, d.S, cw = w.shape
    assert cw == d.C, "channel mismatch"
    d.stride_h, d.stride_w = _pair(stride)
    d.pad_h, d.pad_w = _pair(padding)
    d.opad_h, d.opad_w = _pair(output_padding)
    d.xs = (ctypes.c_longlong * 4)(*_estrides(x))
    d.ws = (ctypes.c_longlong * 4)(*_estrides(w))
    d.os = (ctypes.c_longlong * 4)(*_estrides(out))
    if residual is not None:
        d.rs = (ctypes.c_longlong * 4)(*_estrides(residual))
    d.act = ACT[act]
    rc = lib().oracle_conv_transpose2d(ctypes.byref(d), _ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out))
    assert rc == 0
    return out


def gemm(a, b, bias=None, residual=None, act="none"):
    """C = act(A[M,K] @ B[K,N] + bias + residual), fp32 accumulation (include/tracea.hpp:139-144)."""
    M, K = a.shape
    kb, N = b.shape
    assert kb == K, "inner dimension mismatch"
    c = np.empty((M, N), np.float32)
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np.float32)
    d = _GemmDesc()
    d.M, d.N, d.K = M, N, K
    d.as_ = (ctypes.c_longlong * 2)(*_estrides(a))
    d.bs = (ctypes.c_longlong * 2)(*_estrides(b))
    d.cs = (ctypes.c_longlong * 2)(*_estrides(c))
    if residual is not None:
        d.rs = (ctypes.c_longlong * 2)(*_estrides(residual))
    d.act = ACT[act]
    rc = lib().oracle_gemm(ctypes.byref(d), _ptr(a), _ptr(b), _ptr(bias), _ptr(residual), _ptr(c))
    assert rc == 0
    return c

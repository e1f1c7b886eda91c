"""The reference's Python operator surface for Conv2d, on torch tensors, over the C ABI.

Mirrors (paths relative to the reference project's root):
  * ``tracea.ops.conv2d(x, w, bias, residual, epilogue, stride, padding, dilation)`` with x in
    NHWC and w in KRSC memory (tracea-python/python/tracea/ops.py:39-70);
  * ``Context.conv2d(x, w, o, n, c, h, w_in, k, r, s, stride, pad, dilation, epilogue, bias,
    residual)`` and its epilogue grammar ``"bias+relu"``, ``"bias+residual+relu"``
    (src/interface/python.rs:41-87, 367-462);
  * the NCHW / OIHW call the C++ header documents (include/tracea.hpp:101-105) as ``conv2d_nchw``.

torch is used for device memory and streams only. Every call goes through ``tracea_conv2d`` in
libtracea_b200.so; nothing here computes a convolution itself.
"""
import ctypes

import torch

from . import ffi

_DTYPES = {torch.float32: ffi.DTYPE_FLOAT32, torch.float16: ffi.DTYPE_FLOAT16,
           torch.bfloat16: ffi.DTYPE_BFLOAT16, torch.int32: ffi.DTYPE_INT32, torch.int8: ffi.DTYPE_INT8}

_ACTS = ("relu", "gelu", "silu")


def parse_epilogue(epilogue, bias=None, residual=None):
    """Epilogue string -> TraceaEpilogueKind, with the grammar and the errors of
    src/interface/python.rs:41-87: '+'-separated, case-insensitive ops out of identity, relu, gelu,
    silu, bias, residual; 'bias' / 'residual' without the matching tensor is a ValueError, so is an
    unknown op. The kernel applies bias -> residual -> activation, the order the reference's graph
    fusion produces (tests/fusion_verification.rs:110-170); other orders are rejected."""
    if epilogue is None:
        return ffi.EPILOGUE_IDENTITY
    ops = []
    for part in epilogue.split("+"):
        op = part.strip().lower()
        if op == "identity":
            continue
        if op in _ACTS or op in ("bias", "residual"):
            ops.append(op)
        else:
            raise ValueError("Unknown epilogue op: %s" % part)
    if "bias" in ops and bias is None:
        raise ValueError("Epilogue contains 'bias' but no bias argument provided")
    if "residual" in ops and residual is None:
        raise ValueError("Epilogue contains 'residual' but no reference provided")
    table = {
        (): ffi.EPILOGUE_IDENTITY,
        ("bias",): ffi.EPILOGUE_BIAS_ADD,
        ("relu",): ffi.EPILOGUE_RELU,
        ("gelu",): ffi.EPILOGUE_GELU,
        ("silu",): ffi.EPILOGUE_SILU,
        ("bias", "relu"): ffi.EPILOGUE_BIAS_RELU,
        ("bias", "silu"): ffi.EPILOGUE_BIAS_SILU,
        ("residual",): ffi.EPILOGUE_RESIDUAL,
        ("residual", "relu"): ffi.EPILOGUE_RESIDUAL_RELU,
        ("bias", "residual", "relu"): ffi.EPILOGUE_BIAS_RESIDUAL_RELU,
        ("bias", "residual"): ffi.EPILOGUE_BIAS_RESIDUAL,
    }
    kind = table.get(tuple(ops))
    if kind is None:
        raise ValueError("Unsupported epilogue sequence %r (supported: %s)" % (
            epilogue, ", ".join("+".join(k) or "identity" for k in table)))
    return kind


def _pair(v):
    if isinstance(v, (tuple, list)):
        return int(v[0]), int(v[1])
    return int(v), int(v)


def _device_id(t):
    return t.device.index if t.is_cuda else -1


def _view(t, shape=None, stride=None):
    dt = _DTYPES.get(t.dtype)
    if dt is None:
        raise TypeError("unsupported dtype %s" % t.dtype)
    return ffi.View(t.data_ptr(), t.shape if shape is None else shape, t.stride() if stride is None else stride, dt,
                    t.device.index if t.is_cuda else -1)


def _nchw_view_of_nhwc(t):
    """Logical NCHW view (shape + element strides) of a tensor whose dims are (N, H, W, C)."""
    n, h, w, c = t.shape
    sn, sh, sw, sc = t.stride()
    return _view(t, (n, c, h, w), (sn, sc, sh, sw))


def _stream_of(t):
    return torch.cuda.current_stream(t.device).cuda_stream if t.is_cuda else 0


def conv2d_into(x, w, out, bias=None, residual=None, stride=1, padding=0, dilation=1, groups=1,
                epilogue=ffi.EPILOGUE_IDENTITY, stream=None):
    """out <- epilogue(conv2d(x, w)) with logical NCHW / OIHW tensors of any strides (a
    ``channels_last`` torch tensor is consumed in place). Enqueues on torch's current stream."""
    if stream is None:
        stream = _stream_of(x)
    ffi.conv2d_raw(_view(x), _view(w), _view(bias) if bias is not None else None,
                   _view(residual) if residual is not None else None, _view(out),
                   _pair(stride), _pair(padding), _pair(dilation), groups, epilogue, stream)
    return out


def conv2d_nchw(x, w, bias=None, residual=None, stride=1, padding=0, dilation=1, groups=1, epilogue=None,
                channels_last_out=None):
    """Logical-NCHW convolution (include/tracea.hpp:101-105). The output takes the memory format of
    ``x`` unless ``channels_last_out`` says otherwise."""
    kind = epilogue if isinstance(epilogue, int) else parse_epilogue(epilogue, bias, residual)
    sh, sw = _pair(stride)
    ph, pw = _pair(padding)
    dh, dw = _pair(dilation)
    n, _, h, wi = x.shape
    k, _, r, s = w.shape
    ho = (h + 2 * ph - dh * (r - 1) - 1) // sh + 1
    wo = (wi + 2 * pw - dw * (s - 1) - 1) // sw + 1
    if channels_last_out is None:
        channels_last_out = x.stride(1) == 1 and x.shape[1] > 1
    fmt = torch.channels_last if channels_last_out else torch.contiguous_format
    out = torch.empty((n, k, ho, wo), dtype=x.dtype, device=x.device, memory_format=fmt)
    return conv2d_into(x, w, out, bias, residual, stride, padding, dilation, groups, kind)


def conv2d(x, w, bias=None, residual=None, epilogue=None, stride=1, padding=0, dilation=1):
    """tracea.ops.conv2d: x (N, H, W, C) channels-last, w (K, R, S, C), optional bias (K) and
    residual (N, Ho, Wo, K); returns (N, Ho, Wo, K). Same shape checks and messages as
    tracea-python/python/tracea/ops.py:52-61."""
    if x.ndim != 4 or w.ndim != 4:
        raise ValueError("Expected NHWC input and KRSC weight")
    n_batch, h, w_in, c = x.shape
    k, r, s, c_w = w.shape
    if c != c_w:
        raise ValueError(f"Channel mismatch: x({c}) vs w({c_w})")
    sh, sw = _pair(stride)
    ph, pw = _pair(padding)
    dh, dw = _pair(dilation)
    h_out = (h + 2 * ph - dh * (r - 1) - 1) // sh + 1
    w_out = (w_in + 2 * pw - dw * (s - 1) - 1) // sw + 1
    o = torch.empty((n_batch, h_out, w_out, k), dtype=x.dtype, device=x.device)
    Context().conv2d(x, w, o, n_batch, c, h, w_in, k, r, s, stride=stride, pad=padding, dilation=dilation,
                     epilogue=epilogue, bias=bias, residual=residual)
    return o


def gemm(x, w, bias=None, epilogue=None, residual=None):
    """tracea.ops.gemm (tracea-python/python/tracea/ops.py:12-35): x (M, K) @ w (K, N) -> (M, N) with the conv
    epilogue. Any strides; a ``w`` whose memory is [N][K] (``weight.t()`` of a Linear layer, or the result of
    ``prepack_gemm_b``) is read in place, a row-major one is transposed into scratch on every call."""
    if x.ndim != 2 or w.ndim != 2:
        raise ValueError("Expected 2D tensors: x (M, K), w (K, N)")
    if x.shape[1] != w.shape[0]:
        raise ValueError(f"Inner dimension mismatch: x({x.shape[1]}) vs w({w.shape[0]})")
    kind = parse_epilogue(epilogue, bias, residual)
    out = torch.empty((x.shape[0], w.shape[1]), dtype=x.dtype, device=x.device)
    ffi.gemm_raw(_view(x), _view(w), _view(bias) if bias is not None else None,
                 _view(residual) if residual is not None else None, _view(out), kind, _stream_of(x))
    return out


def conv_transpose2d(x, w, bias=None, residual=None, epilogue=None, stride=1, padding=0, output_padding=0,
                     dilation=1):
    """tracea.ops.conv_transpose2d (tracea-python/python/tracea/ops.py:72-88): x (N, H, W, C), w (K, R, S, C),
    optional bias (K) and residual (N, Ho, Wo, K); returns (N, Ho, Wo, K) with
    Ho = (H-1)*stride - 2*padding + R + output_padding."""
    if x.ndim != 4 or w.ndim != 4:
        raise ValueError("Expected NHWC input and KRSC weight")
    n_batch, h, w_in, c = x.shape
    k, r, s, c_w = w.shape
    if c != c_w:
        raise ValueError(f"Channel mismatch: x({c}) vs w({c_w})")
    sh, sw = _pair(stride)
    ph, pw = _pair(padding)
    oh, ow = _pair(output_padding)
    h_out = (h - 1) * sh - 2 * ph + r + oh
    w_out = (w_in - 1) * sw - 2 * pw + s + ow
    kind = parse_epilogue(epilogue, bias, residual)
    o = torch.empty((n_batch, h_out, w_out, k), dtype=x.dtype, device=x.device)
    ffi.conv_transpose2d_raw(_view(x), _view(w), _view(bias) if bias is not None else None,
                             _view(residual) if residual is not None else None, _view(o), (sh, sw), (ph, pw),
                             (oh, ow), _pair(dilation), 1, kind, _stream_of(x))
    return o


def prepack_conv2d_weight(w):
    """OIHW-shaped weights of any strides -> a tensor of the same logical shape (channels rounded up to 16 bytes)
    whose memory is the dense [K][R][S][C] layout the kernel reads in place (tracea_conv2d_prepack)."""
    lib = ffi.load()
    v = _view(w)
    nbytes = lib.tracea_conv2d_prepack_bytes(v.c)
    shape = (ctypes.c_uint64 * 4)()
    stride = (ctypes.c_int64 * 4)()
    buf = torch.empty(nbytes // w.element_size(), dtype=w.dtype, device=w.device)
    st = lib.tracea_conv2d_prepack(v.c, buf.data_ptr(), nbytes, shape, stride, _stream_of(w))
    if st != ffi.SUCCESS:
        raise ffi.TraceaError(st, ffi.last_error(), "tracea_conv2d_prepack")
    return torch.as_strided(buf, tuple(int(d) for d in shape), tuple(int(d) for d in stride))


def prepack_gemm_b(b):
    """(K, N) matrix of any strides -> a (K, N) tensor whose memory is [N][K] (tracea_gemm_prepack_b)."""
    lib = ffi.load()
    v = _view(b)
    nbytes = lib.tracea_gemm_prepack_b_bytes(v.c)
    stride = (ctypes.c_int64 * 2)()
    buf = torch.empty(nbytes // b.element_size(), dtype=b.dtype, device=b.device)
    st = lib.tracea_gemm_prepack_b(v.c, buf.data_ptr(), nbytes, stride, _stream_of(b))
    if st != ffi.SUCCESS:
        raise ffi.TraceaError(st, ffi.last_error(), "tracea_gemm_prepack_b")
    return torch.as_strided(buf, tuple(b.shape), (int(stride[0]), int(stride[1])))


class Context:
    """Stand-in for the reference's ``tracea.Context`` (src/interface/python.rs:367-462), Conv2d only.
    The reference builds an IR, generates CUDA text and compiles it here; this one forwards to the
    precompiled library."""

    def conv2d(self, x, w, o, n, c, h, w_in, k, r, s, stride=1, pad=0, dilation=1, epilogue=None, bias=None,
               residual=None):
        kind = parse_epilogue(epilogue, bias, residual)
        if tuple(x.shape) != (n, h, w_in, c) or tuple(w.shape) != (k, r, s, c):
            raise ValueError("x must be (n, h, w_in, c) and w must be (k, r, s, c)")
        wk, wr, ws_, wc = w.stride()
        res_view = _nchw_view_of_nhwc(residual) if residual is not None else None
        ffi.conv2d_raw(_nchw_view_of_nhwc(x), _view(w, (k, c, r, s), (wk, wc, wr, ws_)),
                       _view(bias) if bias is not None else None, res_view, _nchw_view_of_nhwc(o),
                       _pair(stride), _pair(pad), _pair(dilation), 1, kind, _stream_of(x))
        return 0

    def synchronize(self):
        torch.cuda.synchronize()

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
    if t.dtype not in _DTYPES:
        raise TypeError("unsupported dtype %s" % t.dtype)
    return ffi.View(t.data_ptr(), tuple(t.shape) if shape is None else shape,
                    tuple(t.stride()) if stride is None else stride, _DTYPES[t.dtype], _device_id(t))


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

"""ctypes binding of the C ABI in include/tracea_b200.h.

The structures repeat the reference's `#[repr(C)]` layouts (tracea-ffi/src/lib.rs:42-71,
include/tracea.hpp:59-82). Loading fails loudly when the compiled library is absent: there is no
Python or CPU fallback behind this module.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtracea_b200.so")

# TraceaStatus (include/tracea.hpp:16-23)
SUCCESS, INVALID_PARAMS, UNSUPPORTED_CONFIG, CUDA_ERROR, CPU_ERROR, UNKNOWN_ERROR = 0, 1, 2, 3, 4, 99
STATUS_NAMES = {0: "SUCCESS", 1: "INVALID_PARAMS", 2: "UNSUPPORTED_CONFIG", 3: "CUDA_ERROR", 4: "CPU_ERROR",
                99: "UNKNOWN_ERROR"}
# TraceaDType (include/tracea.hpp:29-35)
DTYPE_FLOAT32, DTYPE_FLOAT16, DTYPE_BFLOAT16, DTYPE_INT32, DTYPE_INT8 = 0, 1, 2, 3, 4
# TraceaEpilogueKind (include/tracea.hpp:37-47) + the two combined kinds this library adds
(EPILOGUE_IDENTITY, EPILOGUE_BIAS_ADD, EPILOGUE_RELU, EPILOGUE_GELU, EPILOGUE_SILU, EPILOGUE_BIAS_RELU,
 EPILOGUE_BIAS_SILU, EPILOGUE_RESIDUAL, EPILOGUE_RESIDUAL_RELU, EPILOGUE_BIAS_RESIDUAL_RELU,
 EPILOGUE_BIAS_RESIDUAL) = range(11)

EXPORTED_SYMBOLS = (
    "tracea_conv2d", "tracea_conv2d_v0", "tracea_conv2d_noalloc", "tracea_get_last_error", "tracea_clear_error",
    "tracea_version_major", "tracea_version_minor", "tracea_version_patch", "tracea_init",
    "tracea_shutdown", "tracea_b200_device_status", "tracea_b200_launch_count", "tracea_b200_launch_count_of", "tracea_b200_test_hooks", "tracea_b200_pool_stats",
    "tracea_b200_conv_transpose_plan",
    "tracea_gemm", "tracea_conv_transpose2d", "tracea_conv2d_prepack_bytes", "tracea_conv2d_prepack",
    "tracea_gemm_prepack_b_bytes", "tracea_gemm_prepack_b",
)


class TensorView(ctypes.Structure):
    _fields_ = [
        ("ptr", ctypes.c_void_p),
        ("rank", ctypes.c_uint32),
        ("shape", ctypes.POINTER(ctypes.c_uint64)),
        ("stride", ctypes.POINTER(ctypes.c_int64)),
        ("dtype", ctypes.c_int),
        ("device_id", ctypes.c_int32),
    ]


class Conv2dParams(ctypes.Structure):
    _fields_ = [
        ("stride_h", ctypes.c_uint32), ("stride_w", ctypes.c_uint32),
        ("padding_h", ctypes.c_uint32), ("padding_w", ctypes.c_uint32),
        ("dilation_h", ctypes.c_uint32), ("dilation_w", ctypes.c_uint32),
        ("groups", ctypes.c_uint32),
        ("epilogue", ctypes.c_int),
        ("stream", ctypes.c_void_p),
    ]


class Conv2dParamsV0(ctypes.Structure):
    _fields_ = [
        ("stride_h", ctypes.c_uint32), ("stride_w", ctypes.c_uint32),
        ("padding_h", ctypes.c_uint32), ("padding_w", ctypes.c_uint32),
        ("dilation_h", ctypes.c_uint32), ("dilation_w", ctypes.c_uint32),
        ("groups", ctypes.c_uint32),
        ("stream", ctypes.c_void_p),
    ]


class GemmParams(ctypes.Structure):
    _fields_ = [("epilogue", ctypes.c_int), ("stream", ctypes.c_void_p)]


class ConvTranspose2dParams(ctypes.Structure):
    _fields_ = [
        ("stride_h", ctypes.c_uint32), ("stride_w", ctypes.c_uint32),
        ("padding_h", ctypes.c_uint32), ("padding_w", ctypes.c_uint32),
        ("output_padding_h", ctypes.c_uint32), ("output_padding_w", ctypes.c_uint32),
        ("dilation_h", ctypes.c_uint32), ("dilation_w", ctypes.c_uint32),
        ("groups", ctypes.c_uint32),
        ("epilogue", ctypes.c_int),
        ("stream", ctypes.c_void_p),
    ]


class TraceaError(RuntimeError):
    """A non-zero TraceaStatus, carrying the library's last-error text."""

    def __init__(self, status, message, entry="tracea_conv2d"):
        super().__init__("%s failed: %s (%s)" % (entry, message, STATUS_NAMES.get(status, status)))
        self.status = status
        self.message = message


_lib = None


def load():
    """dlopen libtracea_b200.so and declare its prototypes. Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "%s is missing: build it with `python -m tracea_b200.build` (nvcc, sm_100a). "
            "tracea_b200 has no fallback path." % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    lib.tracea_conv2d.argtypes = [TensorView, TensorView, ctypes.POINTER(TensorView), ctypes.POINTER(TensorView),
                                  ctypes.POINTER(TensorView), Conv2dParams]
    lib.tracea_conv2d.restype = ctypes.c_int
    lib.tracea_conv2d_noalloc.argtypes = lib.tracea_conv2d.argtypes
    lib.tracea_conv2d_noalloc.restype = ctypes.c_int
    lib.tracea_conv2d_v0.argtypes = [TensorView, TensorView, ctypes.POINTER(TensorView),
                                     ctypes.POINTER(TensorView), Conv2dParamsV0]
    lib.tracea_conv2d_v0.restype = ctypes.c_int
    lib.tracea_get_last_error.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
    lib.tracea_get_last_error.restype = ctypes.c_int32
    lib.tracea_clear_error.argtypes = []
    lib.tracea_clear_error.restype = None
    for name in ("tracea_version_major", "tracea_version_minor", "tracea_version_patch"):
        getattr(lib, name).argtypes = []
        getattr(lib, name).restype = ctypes.c_uint32
    lib.tracea_init.argtypes = []
    lib.tracea_init.restype = ctypes.c_int
    lib.tracea_shutdown.argtypes = []
    lib.tracea_shutdown.restype = None
    lib.tracea_b200_device_status.argtypes = [ctypes.c_int32]
    lib.tracea_b200_device_status.restype = ctypes.c_uint32
    lib.tracea_b200_pool_stats.argtypes = [ctypes.c_int32, ctypes.POINTER(ctypes.c_uint64), ctypes.c_int32]
    lib.tracea_b200_pool_stats.restype = ctypes.c_int32
    lib.tracea_b200_test_hooks.argtypes = [ctypes.c_int64, ctypes.c_int32]
    lib.tracea_b200_test_hooks.restype = None
    lib.tracea_b200_launch_count_of.argtypes = [ctypes.c_int32]
    lib.tracea_b200_launch_count_of.restype = ctypes.c_uint64
    lib.tracea_b200_launch_count.argtypes = []
    lib.tracea_b200_launch_count.restype = ctypes.c_uint64
    lib.tracea_b200_conv_transpose_plan.argtypes = [ctypes.c_uint32] * 5 + [ctypes.POINTER(ctypes.c_int64)]
    lib.tracea_b200_conv_transpose_plan.restype = ctypes.c_int32
    pv = ctypes.POINTER(TensorView)
    lib.tracea_gemm.argtypes = [TensorView, TensorView, pv, pv, pv, GemmParams]
    lib.tracea_gemm.restype = ctypes.c_int
    lib.tracea_conv_transpose2d.argtypes = [TensorView, TensorView, pv, pv, pv, ConvTranspose2dParams]
    lib.tracea_conv_transpose2d.restype = ctypes.c_int
    lib.tracea_conv2d_prepack_bytes.argtypes = [TensorView]
    lib.tracea_conv2d_prepack_bytes.restype = ctypes.c_uint64
    lib.tracea_conv2d_prepack.argtypes = [TensorView, ctypes.c_void_p, ctypes.c_uint64, ctypes.POINTER(ctypes.c_uint64),
                                          ctypes.POINTER(ctypes.c_int64), ctypes.c_void_p]
    lib.tracea_conv2d_prepack.restype = ctypes.c_int
    lib.tracea_gemm_prepack_b_bytes.argtypes = [TensorView]
    lib.tracea_gemm_prepack_b_bytes.restype = ctypes.c_uint64
    lib.tracea_gemm_prepack_b.argtypes = [TensorView, ctypes.c_void_p, ctypes.c_uint64, ctypes.POINTER(ctypes.c_int64),
                                          ctypes.c_void_p]
    lib.tracea_gemm_prepack_b.restype = ctypes.c_int
    _lib = lib
    return lib


def last_error():
    buf = ctypes.create_string_buffer(1024)
    n = load().tracea_get_last_error(buf, len(buf))
    return buf.raw[:n].decode("utf-8", "replace") if n > 0 else ""


_U64_ARRAYS = {n: ctypes.c_uint64 * n for n in range(0, 9)}
_I64_ARRAYS = {n: ctypes.c_int64 * n for n in range(0, 9)}
_NULL_STRIDE = ctypes.POINTER(ctypes.c_int64)()


class View:
    """Owns the shape/stride arrays a TensorView borrows (the caller-owned arrays of
    include/tracea.hpp:56-66). Construction is on the per-call path of the Python surface, hence the
    pre-built array types."""

    def __init__(self, ptr, shape, stride, dtype, device_id):
        n = len(shape)
        self._shape = _U64_ARRAYS[n](*shape)
        if stride is not None:
            self._stride = _I64_ARRAYS[n](*stride)
            self.c = TensorView(ptr, n, self._shape, self._stride, dtype, device_id)
        else:
            self._stride = None
            self.c = TensorView(ptr, n, self._shape, _NULL_STRIDE, dtype, device_id)


def conv2d_raw(x, w, bias, residual, out, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1,
               epilogue=EPILOGUE_IDENTITY, stream=0, check=True, entry="tracea_conv2d"):
    """Call tracea_conv2d (or the entry point named by ``entry``, which must share its signature)
    with View objects. Returns the status; raises TraceaError when ``check``."""
    lib = load()
    p = Conv2dParams(stride[0], stride[1], padding[0], padding[1], dilation[0], dilation[1], groups,
                     int(epilogue), ctypes.c_void_p(stream))
    st = getattr(lib, entry)(x.c, w.c, ctypes.byref(bias.c) if bias is not None else None,
                           ctypes.byref(residual.c) if residual is not None else None,
                           ctypes.byref(out.c) if out is not None else None, p)
    if check and st != SUCCESS:
        raise TraceaError(st, last_error())
    return st


def _opt(view):
    return ctypes.byref(view.c) if view is not None else None


def gemm_raw(a, b, bias, residual, c, epilogue=EPILOGUE_IDENTITY, stream=0, check=True):
    """Call tracea_gemm with View objects (rank 2; bias rank 1)."""
    st = load().tracea_gemm(a.c, b.c, _opt(bias), _opt(residual), _opt(c),
                            GemmParams(int(epilogue), ctypes.c_void_p(stream)))
    if check and st != SUCCESS:
        raise TraceaError(st, last_error(), "tracea_gemm")
    return st


def conv_transpose2d_raw(x, w, bias, residual, out, stride=(1, 1), padding=(0, 0), output_padding=(0, 0),
                         dilation=(1, 1), groups=1, epilogue=EPILOGUE_IDENTITY, stream=0, check=True):
    """Call tracea_conv_transpose2d with View objects (x [N,H,W,C], w [K,R,S,C], out [N,Ho,Wo,K])."""
    p = ConvTranspose2dParams(stride[0], stride[1], padding[0], padding[1], output_padding[0], output_padding[1],
                              dilation[0], dilation[1], groups, int(epilogue), ctypes.c_void_p(stream))
    st = load().tracea_conv_transpose2d(x.c, w.c, _opt(bias), _opt(residual), _opt(out), p)
    if check and st != SUCCESS:
        raise TraceaError(st, last_error(), "tracea_conv_transpose2d")
    return st


KERNEL_GENERAL, KERNEL_SPLIT_K, KERNEL_RESIDENT_FILTER, KERNEL_LAYOUT, KERNEL_ROW_BAND = range(5)


def launch_count_of(kind):
    """Launches so far of one kind of kernel (KERNEL_* above)."""
    return int(load().tracea_b200_launch_count_of(kind))


def pool_stats(device_id=0, reset_high=False):
    """Scratch-pool byte counters of one device: dict(reserved, reserved_high, used, used_high), or None when
    the device has no pool yet."""
    buf = (ctypes.c_uint64 * 4)()
    rc = load().tracea_b200_pool_stats(device_id, buf, 1 if reset_high else 0)
    if rc < 0:
        raise ValueError("bad arguments")
    if rc == 0:
        return None
    return dict(zip(("reserved", "reserved_high", "used", "used_high"), (int(v) for v in buf)))


def conv_transpose_plan(in_extent, out_extent, filt, stride, padding):
    """Per-phase geometry tracea_conv_transpose2d uses along one axis: a list of dicts, one per phase."""
    buf = (ctypes.c_int64 * (8 * stride))()
    if load().tracea_b200_conv_transpose_plan(in_extent, out_extent, filt, stride, padding, buf) != stride:
        raise ValueError("bad arguments")
    keys = ("a0", "T", "a", "taps", "x_off", "in", "pad_lo", "pad_hi")
    return [dict(zip(keys, buf[8 * i:8 * i + 8])) for i in range(stride)]

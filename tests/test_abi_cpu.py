"""The C-ABI library without a GPU: it loads, exports every symbol the header declares, keeps the
reference's struct layouts, and its validation / error reporting behaves like tracea-ffi's
(tracea-ffi/src/lib.rs:87-109, 144-207). No compute is attempted here."""
import ctypes
import os
import re
import shutil
import subprocess

import numpy as np
import pytest

from tracea_b200 import ffi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "tracea_b200.h")


def _declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tracea_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    assert sorted(ffi.EXPORTED_SYMBOLS) == _declared_functions()


def test_library_exports_every_declared_symbol(lib):
    for name in _declared_functions():
        assert getattr(lib, name) is not None, name


def test_version_is_0_1_0(lib):
    assert (lib.tracea_version_major(), lib.tracea_version_minor(), lib.tracea_version_patch()) == (0, 1, 0)


def test_struct_layouts_match_the_reference_abi():
    # TraceaTensorView: ptr, u32 rank, (pad), shape*, stride*, i32 dtype, i32 device  -> 40 bytes
    assert ctypes.sizeof(ffi.TensorView) == 40
    assert ffi.TensorView.shape.offset == 16 and ffi.TensorView.stride.offset == 24
    assert ffi.TensorView.dtype.offset == 32 and ffi.TensorView.device_id.offset == 36
    # TraceaConv2dParams: 7 x u32, epilogue enum, stream* -> 40 bytes; the older block has no epilogue
    assert ctypes.sizeof(ffi.Conv2dParams) == 40 and ffi.Conv2dParams.stream.offset == 32
    assert ctypes.sizeof(ffi.Conv2dParamsV0) == 40 and ffi.Conv2dParamsV0.stream.offset == 32


def test_header_compiles_as_c_and_cxx(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "tracea_b200.h"\n'
                   "_Static_assert(sizeof(TraceaTensorView) == 40, \"view\");\n"
                   "_Static_assert(sizeof(TraceaConv2dParams) == 40, \"params\");\n"
                   "_Static_assert(TRACEA_EPILOGUE_RESIDUAL_RELU == 8, \"enum\");\n"
                   "int main(void) { return tracea_version_major != 0 ? 0 : 1; }\n")
    inc = os.path.join(ROOT, "include")
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-Wno-address", "-fsyntax-only", "-I", inc, str(src)], check=True)
    cxx = tmp_path / "t.cpp"
    cxx.write_text('#include "tracea_b200.h"\nstatic_assert(sizeof(TraceaTensorView) == 40, "view");\nint main() {}\n')
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-fsyntax-only", "-I", inc, str(cxx)], check=True)


def test_last_error_buffer_contract(lib):
    lib.tracea_clear_error()
    assert lib.tracea_get_last_error(None, 10) == -1
    buf = ctypes.create_string_buffer(8)
    assert lib.tracea_get_last_error(buf, 0) == -1
    assert lib.tracea_get_last_error(buf, 8) == 0 and buf.raw[0] == 0
    # provoke an error, then read it through a buffer that is too short: truncated and NUL-terminated
    x = _view(np.zeros((1, 4, 4, 4), np.float32))
    st = ffi.conv2d_raw(x, x, None, None, x, groups=2, check=False)
    assert st == ffi.UNSUPPORTED_CONFIG
    n = lib.tracea_get_last_error(buf, 8)
    assert n == 7 and buf.raw[7] == 0 and buf.raw[:7] == b"Unsuppo"
    assert ffi.last_error() == "Unsupported groups: 2"
    lib.tracea_clear_error()
    assert ffi.last_error() == ""


_DT = {np.dtype(np.float32): ffi.DTYPE_FLOAT32, np.dtype(np.float16): ffi.DTYPE_FLOAT16,
       np.dtype(np.int32): ffi.DTYPE_INT32, np.dtype(np.int8): ffi.DTYPE_INT8}


def _view(a, device=-1, shape=None, ptr=None):
    v = ffi.View(a.ctypes.data if ptr is None else ptr, a.shape if shape is None else shape,
                 [s // a.itemsize for s in a.strides], _DT[a.dtype], device)
    v._keep = a
    return v


def _xwo(n=1, c=8, h=6, w=6, k=4, r=3, pad=1, dtype=np.float32):
    x = np.zeros((n, c, h, w), dtype)
    wt = np.zeros((k, c, r, r), dtype)
    ho = h + 2 * pad - r + 1
    out = np.zeros((n, k, ho, ho), dtype)
    return x, wt, out


@pytest.mark.parametrize("which", ["x", "w", "out_struct", "out_ptr"])
def test_null_pointers_are_invalid_params(lib, which):
    x, w, o = _xwo()
    vx, vw, vo = _view(x), _view(w), _view(o)
    if which == "x":
        vx = _view(x, ptr=0)
    elif which == "w":
        vw = _view(w, ptr=0)
    elif which == "out_ptr":
        vo = _view(o, ptr=0)
    st = ffi.conv2d_raw(vx, vw, None, None, None if which == "out_struct" else vo, padding=(1, 1), check=False)
    assert st == ffi.INVALID_PARAMS
    assert ffi.last_error() == "Null pointer in input tensors"


def test_groups_not_one_is_unsupported(lib):
    x, w, o = _xwo()
    assert ffi.conv2d_raw(_view(x), _view(w), None, None, _view(o), padding=(1, 1), groups=4,
                          check=False) == ffi.UNSUPPORTED_CONFIG
    assert "groups" in ffi.last_error()


def test_rank_must_be_four(lib):
    x, w, o = _xwo()
    x3 = np.zeros((8, 6, 6), np.float32)
    assert ffi.conv2d_raw(_view(x3), _view(w), None, None, _view(o), padding=(1, 1), check=False) == ffi.INVALID_PARAMS
    assert "4D" in ffi.last_error()


@pytest.mark.parametrize("dtype", [np.int32, np.int8])
def test_integer_dtypes_are_unsupported(lib, dtype):
    x, w, o = _xwo(dtype=dtype)
    assert ffi.conv2d_raw(_view(x), _view(w), None, None, _view(o), padding=(1, 1), check=False) == ffi.UNSUPPORTED_CONFIG


def test_mixed_dtypes_are_unsupported(lib):
    x, w, o = _xwo()
    w16 = w.astype(np.float16)
    assert ffi.conv2d_raw(_view(x), _view(w16), None, None, _view(o), padding=(1, 1), check=False) == ffi.UNSUPPORTED_CONFIG


def test_zero_stride_and_bad_shapes_are_invalid(lib):
    x, w, o = _xwo()
    assert ffi.conv2d_raw(_view(x), _view(w), None, None, _view(o), stride=(0, 1), padding=(1, 1),
                          check=False) == ffi.INVALID_PARAMS
    # out shape must be [N, K, Ho, Wo]
    bad = np.zeros((1, 4, 5, 6), np.float32)
    assert ffi.conv2d_raw(_view(x), _view(w), None, None, _view(bad), padding=(1, 1), check=False) == ffi.INVALID_PARAMS
    assert "does not match expected [1,4,6,6]" in ffi.last_error()
    # channel mismatch between x and w
    w2 = np.zeros((4, 7, 3, 3), np.float32)
    assert ffi.conv2d_raw(_view(x), _view(w2), None, None, _view(o), padding=(1, 1), check=False) == ffi.INVALID_PARAMS
    # filter larger than the padded input
    w3 = np.zeros((4, 8, 9, 9), np.float32)
    assert ffi.conv2d_raw(_view(x), _view(w3), None, None, _view(o), padding=(1, 1), check=False) == ffi.INVALID_PARAMS
    # bias of the wrong length, residual of the wrong shape
    b = np.zeros((5,), np.float32)
    vb = ffi.View(b.ctypes.data, b.shape, [1], ffi.DTYPE_FLOAT32, -1)
    assert ffi.conv2d_raw(_view(x), _view(w), vb, None, _view(o), padding=(1, 1), epilogue=ffi.EPILOGUE_BIAS_ADD,
                          check=False) == ffi.INVALID_PARAMS
    assert ffi.conv2d_raw(_view(x), _view(w), None, _view(bad), _view(o), padding=(1, 1),
                          epilogue=ffi.EPILOGUE_RESIDUAL, check=False) == ffi.INVALID_PARAMS
    # unknown epilogue kind
    assert ffi.conv2d_raw(_view(x), _view(w), None, None, _view(o), padding=(1, 1), epilogue=77,
                          check=False) == ffi.INVALID_PARAMS


def test_tensors_must_share_a_device(lib):
    x, w, o = _xwo()
    assert ffi.conv2d_raw(_view(x, device=0), _view(w, device=-1), None, None, _view(o, device=0),
                          padding=(1, 1), check=False) == ffi.INVALID_PARAMS


def test_empty_batch_is_a_no_op(lib):
    x, w, o = _xwo()
    st = ffi.conv2d_raw(_view(x, shape=(0, 8, 6, 6)), _view(w), None, None, _view(o, shape=(0, 4, 6, 6)),
                        padding=(1, 1), check=False)
    assert st == ffi.SUCCESS


def test_a_valid_call_without_a_gpu_fails_loudly(lib):
    """There is no CPU compute path behind the ABI: with no CUDA device the call must report an
    error status, never produce numbers."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    x, w, o = _xwo()
    o[:] = 7.0
    st = ffi.conv2d_raw(_view(x), _view(w), None, None, _view(o), padding=(1, 1), check=False)
    assert st == ffi.CUDA_ERROR
    assert ffi.last_error() != ""
    assert (o == 7.0).all()
    assert lib.tracea_init() == -1


def test_five_argument_form_validates_like_the_six_argument_form(lib):
    x, w, o = _xwo()
    p = ffi.Conv2dParamsV0(1, 1, 1, 1, 1, 1, 3, None)
    vo = _view(o)
    st = lib.tracea_conv2d_v0(_view(x).c, _view(w).c, None, ctypes.byref(vo.c), p)
    assert st == ffi.UNSUPPORTED_CONFIG


def test_last_error_is_thread_local(lib):
    import threading
    x, w, o = _xwo()
    ffi.conv2d_raw(_view(x), _view(w), None, None, _view(o), groups=2, check=False)
    seen = {}

    def other():
        seen["msg"] = ffi.last_error()

    t = threading.Thread(target=other)
    t.start()
    t.join()
    assert seen["msg"] == "" and ffi.last_error() == "Unsupported groups: 2"


# the reference checkout, when present, sits next to this repository (or where TRACEA_REFERENCE_ROOT points)
_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_HPP = os.path.join(os.environ.get("TRACEA_REFERENCE_ROOT", os.path.join(os.path.dirname(_REPO), "reference")),
                       "include", "tracea.hpp")


@pytest.mark.skipif(not os.path.exists(REF_HPP) or shutil.which("g++") is None,
                    reason="the reference checkout is not present on this machine")
def test_reference_header_links_against_this_library(tmp_path, lib):
    """A caller written against the reference's own, unmodified include/tracea.hpp links and runs
    against libtracea_b200.so (drop-in check; the header is read in place, not copied)."""
    src = tmp_path / "caller.cpp"
    src.write_text(r'''
#include <cstdio>
#include <tracea.hpp>
int main() {
  std::vector<float> x(1 * 8 * 6 * 6), w(4 * 8 * 3 * 3), o(1 * 4 * 6 * 6);
  tracea::TensorView tx(x.data(), {1, 8, 6, 6}, tracea::DType::Float32);
  tracea::TensorView tw(w.data(), {4, 8, 3, 3}, tracea::DType::Float32);
  tracea::TensorView to(o.data(), {1, 4, 6, 6}, tracea::DType::Float32);
  tracea::Conv2dParams p;
  p.padding_h = p.padding_w = 1;
  p.groups = 2;  // rejected by validation, with or without a GPU
  int caught = 0;
  try {
    tracea::conv2d(tx, tw, nullptr, nullptr, to, p);
  } catch (const std::runtime_error& e) {
    std::printf("%s\n", e.what());
    ++caught;
  }
  // the GEMM and ConvTranspose2d wrappers of the same header resolve against this library too
  std::vector<float> a(4 * 8), b(7 * 6), c(4 * 6);
  tracea::TensorView ta(a.data(), {4, 8}, tracea::DType::Float32);
  tracea::TensorView tb(b.data(), {7, 6}, tracea::DType::Float32);     // inner dimension mismatch
  tracea::TensorView tc(c.data(), {4, 6}, tracea::DType::Float32);
  try {
    tracea::gemm(ta, tb, nullptr, nullptr, tc, tracea::GemmParams());
  } catch (const std::runtime_error& e) {
    std::printf("%s\n", e.what());
    ++caught;
  }
  tracea::ConvTranspose2dParams tp;
  tp.groups = 2;
  try {
    tracea::conv_transpose2d(tx, tw, nullptr, nullptr, to, tp);
  } catch (const std::runtime_error& e) {
    std::printf("%s\n", e.what());
    ++caught;
  }
  return caught == 3 ? 0 : 1;
}
''')
    exe = tmp_path / "caller"
    libdir = os.path.dirname(ffi.LIB_PATH)
    subprocess.run(["g++", "-std=c++17", "-I", os.path.dirname(REF_HPP), str(src), "-o", str(exe),
                    "-L", libdir, "-ltracea_b200", "-Wl,-rpath," + libdir, "-Wl,--allow-shlib-undefined"], check=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True)
    assert res.returncode == 0
    assert res.stdout.strip().splitlines() == [
        "tracea::conv2d failed: Unsupported groups: 2",
        "tracea::gemm failed: Inner dimension mismatch: a is [4,8], b is [7,6]",
        "tracea::conv_transpose2d failed: Unsupported groups: 2",
    ]

"""TEST INFRASTRUCTURE ONLY.  ctypes access to oracle/_ref/libfp6ref.so - the reference's own host
code (quantize / prepacking / dequantize), compiled unmodified by oracle/build_ref.py.  Used to
pin the NumPy restatement in oracle/formats.py, to generate the golden vectors under
tests/golden/, and as the "reference" CPU baseline timed by the benchmark.  Shapes follow the
reference's torch bindings (fp6_marlin/pybind.cpp:18-87).
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libfp6ref.so")
_lib = None


def available() -> bool:
    return os.path.isfile(_LIB_PATH)


def _load():
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(_LIB_PATH)
        vp, sz = ctypes.c_void_p, ctypes.c_size_t
        lib.ref_quantize_fp6.argtypes = [vp, vp, sz, sz]
        lib.ref_prepack_fp6.argtypes = [vp, vp, sz, sz]
        lib.ref_dequant_fp6.argtypes = [vp, vp, vp, sz, sz]
        for f in (lib.ref_quantize_fp6, lib.ref_prepack_fp6, lib.ref_dequant_fp6):
            f.restype = ctypes.c_int
        _lib = lib
    return _lib


def _ptr(a: np.ndarray):
    return ctypes.c_void_p(a.ctypes.data)


def quantize(w: np.ndarray) -> np.ndarray:
    """(a, b) fp16 -> (b, a*3/16) int32, as ``fp6_marlin.quantize`` (pybind.cpp:42-59)."""
    assert w.dtype == np.float16
    a, b = w.shape
    assert a % 256 == 0 and b % 256 == 0
    w = np.ascontiguousarray(w)
    out = np.empty((b, a * 3 // 16), dtype=np.int32)
    # pybind.cpp:57 calls weight_prepacking_fp16_to_fp6(ptr, out, IC, OC) with IC=b, OC=a
    rc = _load().ref_quantize_fp6(_ptr(w), _ptr(out), b, a)
    if rc:
        raise ValueError("Input value out of range for FP6.")
    return out


def prepacking(fp6: np.ndarray) -> np.ndarray:
    """(n, k*3/16) int32 -> (k*3/32, 2n) int32, as ``fp6_marlin.prepacking`` (pybind.cpp:18-31)."""
    assert fp6.dtype == np.int32
    n = fp6.shape[0]
    k = fp6.shape[1] * 16 // 3
    assert n % 256 == 0 and k % 256 == 0
    fp6 = np.ascontiguousarray(fp6)
    out = np.empty((k * 3 // 32, n * 2), dtype=np.int32)
    _load().ref_prepack_fp6(_ptr(fp6), _ptr(out), n, k)
    return out


def dequantize(fp6: np.ndarray, scale: np.ndarray) -> np.ndarray:
    """(n, k*3/16) int32 + (n,) fp16 -> (n, k) fp16, as ``fp6_marlin.dequantize`` (pybind.cpp:70-87)."""
    assert fp6.dtype == np.int32 and scale.dtype == np.float16
    n = fp6.shape[0]
    k = fp6.shape[1] * 16 // 3
    fp6 = np.ascontiguousarray(fp6)
    scale = np.ascontiguousarray(scale)
    out = np.empty((n, k), dtype=np.float16)
    _load().ref_dequant_fp6(_ptr(fp6), _ptr(scale), _ptr(out), n, k)
    return out

"""ctypes binding of libfp6m.so (the C ABI declared in include/fp6m.h).

The library is built in-tree by ``python fp6_marlin_b200/build.py``.  There is no fallback: if the
shared library is missing, importing this module raises, and every GPU entry point raises when
the CUDA call fails.
"""
from __future__ import annotations

import ctypes
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
# FP6M_LIB selects another build of the same library (e.g. the timeline build, see build.py --trace)
LIB_PATH = os.environ.get("FP6M_LIB") or os.path.join(_PKG_DIR, "libfp6m.so")

OK, ERR_PROB_SHAPE, ERR_KERN_SHAPE, ERR_VALUE_RANGE, ERR_BAD_ARG = 0, 1, 2, 3, 4
ERR_WORKSPACE, ERR_SCRATCH, ERR_CUDA, ERR_TIMEOUT = 5, 6, 7, 8
LAYOUT_REFERENCE, LAYOUT_B200 = 0, 1
EPILOGUE_NONE, EPILOGUE_SILU_MUL, EPILOGUE_RESIDUAL = 0, 1, 2

# every symbol include/fp6m.h declares, with its ctypes signature
_vp, _sz, _i, _i64 = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int64
SIGNATURES = {
    "fp6m_quantize_fp6": (_i, [_vp, _vp, _sz, _sz]),
    "fp6m_encode_fp6": (_i, [_vp, _vp, _sz]),
    "fp6m_prepack_fp6": (_i, [_vp, _vp, _sz, _sz]),
    "fp6m_dequant_fp6": (_i, [_vp, _vp, _vp, _sz, _sz]),
    "fp6m_b200_weight_bytes": (_i64, [_i, _i, _i]),
    "fp6m_b200_scale_count": (_i64, [_i, _i, _i, _i]),
    "fp6m_pack_b200": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp]),
    "fp6m_unpack_b200": (_i, [_vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "fp6m_unpack_reference": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "fp6m_repack_from_reference": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp]),
    "fp6m_schedule": (_i, [_i, _i, _i, _i, _i, _vp]),
    "fp6m_mul_scratch_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "fp6m_mul_launches": (_i, [_i, _i, _i, _i, _i, _vp]),
    "fp6m_mul": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp, _sz, _vp, _sz, _i, _vp,
                      _i, _i, _i, _i, _i, _i, _i, _vp]),
    "fp6m_mul_fused": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp, _sz, _vp, _sz, _i, _vp,
                            _i, _i, _i, _i, _i, _i, _i, _vp, _i, _vp]),
    "fp6m_mul_static_scratch": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp, _sz, _i, _vp,
                                     _i, _i, _i, _i, _i, _i, _i, _vp]),
    "fp6m_dump_operands": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "fp6m_mul_scatter": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                        ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t,
                                        ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p] + [ctypes.c_int] * 7 + [ctypes.c_void_p]),
    "fp6m_peer_alloc": (ctypes.c_int, [ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]),
    "fp6m_peer_open": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]),
    "fp6m_peer_close": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int]),
    "fp6m_peer_free": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int]),
    "fp6m_peer_signal": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]),
    "fp6m_peer_signal_wait": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]),
    "fp6m_peer_wait": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]),
    "fp6m_set_peer_wait_polls": (ctypes.c_int, [ctypes.c_int]),
    "fp6m_debug_busy_kernel": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]),
    "fp6m_encode_fp6_device": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]),
    "fp6m_pack_b200_device": (ctypes.c_int, [ctypes.c_void_p] * 4 + [ctypes.c_int] * 4 + [ctypes.c_void_p] * 2 + [ctypes.c_int, ctypes.c_void_p]),
    "fp6m_set_launch_overlap": (ctypes.c_int, [ctypes.c_int]),
    "fp6m_set_ordered_sums": (ctypes.c_int, [ctypes.c_int]),
    "fp6m_last_cuda_error": (ctypes.c_char_p, []),
    "fp6m_version": (ctypes.c_char_p, []),
}


def _load() -> ctypes.CDLL:
    if not os.path.isfile(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python fp6_marlin_b200/build.py` "
            "(there is no fallback implementation)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = _load()


def last_cuda_error() -> str:
    return lib.fp6m_last_cuda_error().decode()

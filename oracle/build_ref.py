"""TEST INFRASTRUCTURE ONLY - builds the checker, is never imported by the product path.

Compiles the reference's own host sources (fp6_marlin/weight_quant.cpp and
fp6_marlin/weight_prepacking.cpp, read where they lie in the reference checkout) together with
oracle/ref_shim.cpp into oracle/_ref/libfp6ref.so.  No reference source is copied into this
repository; only the built library lands in oracle/_ref/ (git-ignored).

The two extra ``-include`` flags supply headers the reference forgets (<cstdint>, <stdexcept>,
<cmath>) under g++ 13; nothing else about the sources is changed.

Usage:  python oracle/build_ref.py [path-to-reference-checkout]
(default: $FP6M_REFERENCE_DIR, else the directory "reference" beside this repository)
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT_LIB = os.path.join(OUT_DIR, "libfp6ref.so")
# the reference checkout: $FP6M_REFERENCE_DIR, else a directory "reference" beside this repository
DEFAULT_REFERENCE = os.environ.get("FP6M_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
CUDA_INCLUDE = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")


def reference_sources(ref_dir: str) -> list[str]:
    return [
        os.path.join(ref_dir, "fp6_marlin", "weight_quant.cpp"),
        os.path.join(ref_dir, "fp6_marlin", "weight_prepacking.cpp"),
    ]


def build(ref_dir: str = DEFAULT_REFERENCE, force: bool = False) -> str | None:
    """Build oracle/_ref/libfp6ref.so; returns its path, or None if the reference is absent."""
    srcs = reference_sources(ref_dir)
    if not all(os.path.isfile(s) for s in srcs):
        return OUT_LIB if os.path.isfile(OUT_LIB) else None
    shim = os.path.join(HERE, "ref_shim.cpp")
    if not force and os.path.isfile(OUT_LIB):
        newest = max(os.path.getmtime(p) for p in srcs + [shim])
        if os.path.getmtime(OUT_LIB) >= newest:
            return OUT_LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = [
        "g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-w",
        "-I", CUDA_INCLUDE,
        "-include", "cstdint", "-include", "stdexcept", "-include", "cmath",
        *srcs, shim, "-o", OUT_LIB,
    ]
    subprocess.run(cmd, check=True)
    return OUT_LIB


if __name__ == "__main__":
    path = build(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_REFERENCE, force=True)
    print(path if path else "reference sources not found; nothing built")

"""Builds fp6_marlin_b200/libfp6m.so in-tree with nvcc for sm_100a (no GPU needed to compile).

Usage:  python fp6_marlin_b200/build.py [--force] [--verbose] [--trace]   (run as a script: it must
work before the package itself can be imported)
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libfp6m.so")
OBJ_DIR = os.path.join(PKG_DIR, "build")

CUDA_SOURCES = ["c_api.cu", "gemm_tc5.cu", "gemm_wide.cu", "dump_operands.cu", "prep_gpu.cu", "peer.cu"]
HOST_SOURCES = ["host_pack.cpp"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = os.path.join(cuda_home, "bin", "nvcc")
    return cand if os.path.isfile(cand) else (shutil.which("nvcc") or "nvcc")


def _sources() -> list[str]:
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(os.path.dirname(PKG_DIR), "include", "fp6m.h"))
    return [os.path.join(CSRC, f) for f in CUDA_SOURCES + HOST_SOURCES] + headers


def needs_build() -> bool:
    if not os.path.isfile(LIB_PATH):
        return True
    lib_time = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(s) > lib_time for s in _sources())


def build(force: bool = False, verbose: bool = False, trace: bool = False) -> str:
    """Compile every source to an object and link the shared library; returns its path.
    ``trace=True`` builds libfp6m_trace.so instead: the same library with the in-kernel timeline of
    csrc/trace.cuh compiled in (read by ``python -m fp6_marlin_b200.timeline``)."""
    lib_path = os.path.join(PKG_DIR, "libfp6m_trace.so") if trace else LIB_PATH
    obj_dir = OBJ_DIR + ("_trace" if trace else "")
    if not force and not trace and not needs_build():
        return lib_path
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = _nvcc()
    objs, procs = [], []
    log = []
    for src in CUDA_SOURCES + HOST_SOURCES:
        obj = os.path.join(obj_dir, os.path.splitext(src)[0] + ".o")
        objs.append(obj)
        cmd = [nvcc, *NVCC_FLAGS, *(["-DFP6M_TRACE"] if trace else []), "-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, proc in procs:
        out, _ = proc.communicate()
        log.append(f"==== {src}\n{out}")
        failed |= proc.returncode != 0
    text = "\n".join(log)
    with open(os.path.join(obj_dir, "ptxas.log"), "w") as f:
        f.write(text)
    if failed or verbose:
        print(text)
    if failed:
        raise RuntimeError("nvcc failed; see output above")
    subprocess.run([nvcc, "-shared", "-o", lib_path, *objs, "-lcudart"], check=True)
    return lib_path


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, trace="--trace" in sys.argv))

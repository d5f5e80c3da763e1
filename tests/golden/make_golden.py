"""Generates the golden vectors in this folder from the REFERENCE ITSELF.  Run it in a container
that has the reference checkout; the fixtures it writes are committed, this script is what made
them, and nothing at test time needs the reference checkout.

Two sources, both unmodified reference code:
  * the reference's host C++ (quantize / prepacking / dequantize), through oracle/_ref
    (built by oracle/build_ref.py from the reference's own sources);
  * the reference's Python weight generators ``gen_int4_weight`` / ``gen_fp6_weight`` /
    ``gen_mixed_weight`` (test.py:13-152), imported from the checkout with the ``fp6_marlin`` module
    replaced by a stub over oracle/_ref and the device set to cpu.

Usage:  python tests/golden/make_golden.py [path-to-reference-checkout]
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import build_ref, ref_lib  # noqa: E402


def _stub_fp6_marlin():
    m = types.ModuleType("fp6_marlin")
    m.quantize = lambda t: torch.from_numpy(ref_lib.quantize(t.contiguous().numpy()))
    m.prepacking = lambda t: torch.from_numpy(ref_lib.prepacking(t.contiguous().numpy()))
    m.dequantize = lambda t, s: torch.from_numpy(
        ref_lib.dequantize(t.contiguous().numpy(), s.contiguous().numpy()))
    m.mul = None
    sys.modules["fp6_marlin"] = m


def _import_reference_test(ref_dir: str):
    spec = importlib.util.spec_from_file_location("reference_test", os.path.join(ref_dir, "test.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.DEV = torch.device("cpu")
    return mod


def main(ref_dir: str) -> None:
    assert build_ref.build(ref_dir) is not None, "reference checkout not found"
    _stub_fp6_marlin()
    ref_test = _import_reference_test(ref_dir)

    # 1. all 64 codes -> fp16, through the reference dequantiser with unit scale: one row of a
    #    64 x 64 matrix holds every code once (dequantMatrix asserts multiples of 64).
    codes = np.tile(np.arange(64, dtype=np.uint8), (64, 1))
    from oracle import formats
    stream = formats.fp6_pack_stream(codes).view(np.int32)
    table = ref_lib.dequantize(stream, np.ones(64, dtype=np.float16))[0]
    np.save(os.path.join(HERE, "fp6_code_table_fp16.npy"), table.view(np.uint16))

    # 2. quantize -> dequantize -> prepacking of a seeded 256 x 256 fake-quantised matrix.
    rng = np.random.default_rng(20240607)
    w = (rng.standard_normal((256, 256)) * 6.0).astype(np.float16)
    w = np.where(np.abs(w) < np.float16(0.0625), np.float16(0), w)
    w = np.clip(w, np.float16(-28), np.float16(28)).astype(np.float16)
    s = (rng.uniform(0.001, 0.05, size=256)).astype(np.float16)
    q = ref_lib.quantize(w)
    np.savez_compressed(
        os.path.join(HERE, "fp6_host_256x256.npz"),
        w=w.view(np.uint16), s=s.view(np.uint16), quantized=q,
        dequantized=ref_lib.dequantize(q, s).view(np.uint16), prepacked=ref_lib.prepacking(q))

    # 3. the reference's own generators (test.py) on seeded weights: INT4-only, all-FP6 and mixed.
    #    gen_mixed_weight draws its weights with torch.randn as its first action, so seeding, drawing
    #    the same tensor here, and seeding again records the generator's input beside its outputs.
    np.random.seed(0)
    out = {}
    cases = {"int4": (128, 256, -1), "fp6": (256, 256, 256), "mixed": (256, 512, 256)}
    for seed, (name, (k, n, qc)) in enumerate(cases.items()):
        torch.manual_seed(seed)
        out[f"{name}_w"] = torch.randn((k, n), dtype=torch.half, device="cpu").numpy().view(np.uint16)
        torch.manual_seed(seed)
        w_ref, packed, sc = ref_test.gen_mixed_weight(k, n, qc)
        out[f"{name}_shape"] = np.array([k, n, qc], dtype=np.int32)
        out[f"{name}_wref"] = w_ref.numpy().view(np.uint16)
        out[f"{name}_packed"] = packed.numpy()
        out[f"{name}_s"] = sc.numpy().view(np.uint16)
    np.savez_compressed(os.path.join(HERE, "reference_generators.npz"), **out)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else build_ref.DEFAULT_REFERENCE)

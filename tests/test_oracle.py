"""Pins the oracle (oracle/formats.py): against the golden vectors generated from the reference
itself (tests/golden/make_golden.py) and, where the compiled reference host code is present
(oracle/_ref), against that code on fresh seeded inputs."""
import os

import numpy as np
import pytest

from oracle import formats as F
from oracle import ref_lib


def _h(bits):
    return np.asarray(bits).view(np.float16)


def test_code_table_matches_reference(golden_dir):
    table = np.load(os.path.join(golden_dir, "fp6_code_table_fp16.npy"))
    ours = F.fp6_code_to_fp16_bits(np.arange(64, dtype=np.uint8))
    assert np.array_equal(ours, table)
    # known answers: largest value 28, smallest subnormal 0.0625, exponent 7 is an ordinary value
    vals = _h(ours).astype(np.float32)
    assert vals[0b011111] == 28.0 and vals[0b000001] == 0.0625 and vals[0b111111] == -28.0
    assert vals[0b001100] == 1.0


def test_host_functions_match_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "fp6_host_256x256.npz"))
    w, s = _h(g["w"]), _h(g["s"])
    q = F.fp6_quantize(w)
    assert np.array_equal(q, g["quantized"])
    assert np.array_equal(F.fp6_dequant(q, s).view(np.uint16), g["dequantized"])
    assert np.array_equal(F.fp6_prepack_reference(q), g["prepacked"])
    codes = F.fp6_unpack_reference(g["prepacked"], 256, 256)
    assert np.array_equal(codes.T, F.fp6_unpack_stream(q.view(np.uint8).reshape(256, -1)))


@pytest.mark.parametrize("name", ["int4", "fp6", "mixed"])
def test_generators_match_reference_test_script(golden_dir, name):
    """gen_int4_weight / gen_fp6_weight / gen_mixed_weight of the reference's test.py, restated."""
    g = np.load(os.path.join(golden_dir, "reference_generators.npz"))
    k, n, qc = (int(x) for x in g[f"{name}_shape"])
    w = _h(g[f"{name}_w"])
    qc = max(qc, 0)
    refs, packed, scales = [], [], []
    if n - qc:
        q, s, deq = F.int4_quantize_per_channel(w[:, : n - qc])
        refs.append(deq)
        packed.append(F.int4_pack_reference(q).reshape(-1))
        scales.append(F.permute_scales_reference(s))
    if qc:
        x, s = F.fp6_fake_quantize(w[:, n - qc:])
        stream = F.fp6_quantize(x)                      # as test.py:32 calls it: memory as it lies
        refs.append(F.fp6_dequant(stream, s).T)
        packed.append(F.fp6_prepack_reference(stream).reshape(-1))
        scales.append(F.permute_scales_reference(s))
    assert np.array_equal(np.concatenate(refs, axis=1).view(np.uint16), g[f"{name}_wref"])
    assert np.array_equal(np.concatenate(packed), g[f"{name}_packed"].reshape(-1))
    assert np.array_equal(np.concatenate(scales).view(np.uint16), g[f"{name}_s"])


def test_truncation_and_range_rules():
    # truncation toward zero: 1.249 -> 1.0, 1.25 -> 1.25; subnormals shift without rounding
    vals = np.array([1.249, 1.25, 0.1874, 0.07, 27.9, -3.9], dtype=np.float16)
    got = _h(F.fp6_code_to_fp16_bits(F.fp6_encode(vals))).astype(np.float32)
    assert got.tolist() == [1.0, 1.25, 0.125, 0.0625, 24.0, -3.5]
    for bad in (0.03, 28.5, -40.0):
        with pytest.raises(ValueError):
            F.fp6_encode(np.array([bad], dtype=np.float16))
    with pytest.raises(ValueError):
        F.fp6_encode(np.zeros(4, dtype=np.float32))


def test_reference_layout_round_trips():
    rng = np.random.default_rng(3)
    q = rng.integers(0, 16, size=(64, 128), dtype=np.uint8)
    assert np.array_equal(F.int4_unpack_reference(F.int4_pack_reference(q), 64, 128), q)
    s = rng.standard_normal(64).astype(np.float16)
    assert np.array_equal(F.unpermute_scales_reference(F.permute_scales_reference(s)), s)


@pytest.mark.skipif(not ref_lib.available(), reason="oracle/_ref not built (no reference checkout)")
def test_against_compiled_reference_fresh_inputs():
    rng = np.random.default_rng(11)
    for (a, b) in [(256, 256), (512, 256)]:
        w = rng.uniform(-28, 28, size=(a, b)).astype(np.float16)
        w = np.where(np.abs(w) < np.float16(0.0625), np.float16(0), w).astype(np.float16)
        q_ref = ref_lib.quantize(w)
        assert np.array_equal(q_ref, F.fp6_quantize(w))
        s = rng.uniform(0.001, 2.0, size=q_ref.shape[0]).astype(np.float16)
        assert np.array_equal(ref_lib.dequantize(q_ref, s).view(np.uint16), F.fp6_dequant(q_ref, s).view(np.uint16))
        assert np.array_equal(ref_lib.prepacking(q_ref), F.fp6_prepack_reference(q_ref))
    with pytest.raises(ValueError):
        ref_lib.quantize(np.full((256, 256), 30.0, dtype=np.float16))

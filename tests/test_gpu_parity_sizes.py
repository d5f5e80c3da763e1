"""GPU parity at the sizes of the benchmark configurations, through the C ABI behind the Python API.

  * the compute-bound geometry (K = 16384) with more rows than one launch covers, so that the host
    dispatcher's loop over launches (offsets of A and C, ragged last launch) runs;
  * every INT4 code and every FP6 code in every position of a 128-row block, through the GEMM kernels
    themselves (one-hot activation rows return the dequantised weights exactly);
  * the single-GPU sweep layer K = N = 8192 for every M of the sweep, the Llama-2-7B gate_up layer and
    a Llama-2-70B down-projection shard, all against the oracle (oracle/formats.py), not against
    anything the product computes.

Tolerance for the GEMMs: relative Frobenius error <= 1e-3 against the fp32-accumulated product of the
oracle's dequantised weights; the one-hot cases are exact.
"""
import numpy as np
import pytest
import torch

import fp6_marlin_b200 as fm
from fp6_marlin_b200 import synth
from oracle import formats as F

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _dev():
    assert torch.cuda.is_available(), "these tests need a CUDA GPU"
    return torch.device("cuda:0")


def _oracle_weight(w: torch.Tensor, qc: int, gs: int) -> np.ndarray:
    """W_deq by the oracle's rules, from the fp16 weights (columns [INT4 | FP6])."""
    k, n = w.shape
    nq = max(qc, 0)
    parts = []
    if n - nq:
        fn = (lambda x: F.int4_quantize_group(x, 128)) if gs > 0 else F.int4_quantize_per_channel
        parts.append(fn(w[:, : n - nq].numpy())[2])
    if nq:
        parts.append(F.fp6_codes_and_dequant(w[:, n - nq:].numpy())[2])
    return np.concatenate(parts, axis=1)


def _mul(a, ww, m, n, qc, gs, dev):
    c = torch.zeros((m, n), dtype=torch.float16, device=dev)
    workspace = torch.zeros(max(n // 128 * 16, 16), dtype=torch.int32, device=dev)
    fm.mul(a, ww.B, c, ww.s, workspace, qc, group_size=gs, layout="b200")
    torch.cuda.synchronize()
    assert fm.device_status(dev) == 0
    return c


@pytest.mark.parametrize("qc", [0, 128, 256, 512])
def test_compute_bound_geometry_with_several_launches(qc):
    """K = 16384: one launch covers 2048 rows of A (eight 256-row tiles), so M = 2304 is two launches with a ragged
    last one, M = 4096 two full ones and M = 4400 three.  Checked on a subset of rows that touches every launch and
    256-row tile edges."""
    dev = _dev()
    k, n, gs = 16384, 1024, 128
    w = synth.make_weight_fp16(k, n, qc, seed=40 + qc)
    ww = fm.make_w46_weight(w, qc if qc else -1, gs, keep_dequantized=False).to(dev)
    w_deq = _oracle_weight(w, qc, gs)
    for m in (1024, 2304, 4096, 4400):
        a = synth.make_activations(m, k, seed=m)
        c = _mul(a.to(dev), ww, m, n, qc if qc else -1, gs, dev).cpu().numpy().astype(np.float32)
        rows = sorted({0, 1, 255, 256, 511, 1023, 1024 % m, 1025 % m, 2047 % m, 2048 % m, 2303 % m, 4095 % m, 4096 % m, m - 257, m - 2, m - 1})
        c_ref = F.gemm_reference(a.numpy()[rows], w_deq)
        err = F.rel_frobenius(c[rows], c_ref)
        assert err <= TOL, (qc, m, err)


def test_one_ragged_256_row_tile_on_a_large_layer():
    """129 to 256 rows run in the kernel for more than 128 rows only on a layer with many blocks per CTA (on a
    smaller one two launches of the other kernel are faster): K = 16384, N = 7424 has 58 x 128 blocks.  Checked on
    four strips of columns (first, middle and last INT4 strip, the FP6 strips) against the oracle."""
    dev = _dev()
    k, n, qc, gs = 16384, 7424, 256, 128
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    w = synth.make_weight_fp16(k, n, qc, seed=77)
    ww = fm.make_w46_weight(w, qc, gs, keep_dequantized=False, quant_device=dev)
    cols = np.r_[0:128, 3712:3840, 7040:7168, 7168:7424]
    w_deq = _oracle_weight(w[:, cols], qc, gs)
    for m in (130, 200, 256):
        assert fm.launch_plan(m, n, k, qc, sms) == (1, True)
        a = synth.make_activations(m, k, seed=m)
        c = _mul(a.to(dev), ww, m, n, qc, gs, dev).cpu().numpy().astype(np.float32)
        err = F.rel_frobenius(c[:, cols], F.gemm_reference(a.numpy(), w_deq))
        assert err <= TOL, (m, err)
    assert fm.launch_plan(200, 8192, 8192, 256, sms) == (2, False)      # few blocks per CTA: two launches of 128 rows
    assert fm.launch_plan(300, 8192, 8192, 256, sms) == (1, True)


def _all_codes_problem(k, n4, n6, gs, seed):
    """Codes chosen so that every INT4 code and every FP6 code occurs at every row position of a 128-row
    block (checked), random fp16 scales; returns packed tensors and the oracle's dequantised weights."""
    rng = np.random.default_rng(seed)
    kk = np.arange(k)[:, None]
    q4 = ((kk // 128) + 3 * (kk % 128) + 5 * np.arange(n4)[None, :]) % 16
    c6 = ((kk // 128) * 8 + 7 * (kk % 128) + 11 * np.arange(n6)[None, :]) % 64
    for codes, ncodes in ((q4, 16), (c6, 64)):
        seen = np.zeros((128, ncodes), dtype=bool)
        seen[(kk % 128).repeat(codes.shape[1], axis=1).ravel(), codes.ravel()] = True
        assert seen.all()
    groups = k // 128 if gs > 0 else 1
    s4 = (rng.uniform(0.004, 0.03, size=(groups, n4))).astype(np.float16)
    s6 = (rng.uniform(0.002, 0.02, size=(n6,))).astype(np.float16)
    B, s = fm.pack_b200(torch.from_numpy(q4.astype(np.uint8)), torch.from_numpy(c6.astype(np.uint8)),
                        torch.from_numpy(s4.reshape(-1) if gs <= 0 else s4), torch.from_numpy(s6), k, n4 + n6, n6, gs)
    w4 = F.int4_dequant(q4.astype(np.uint8), s4 if gs > 0 else s4.reshape(-1), gs)
    v6 = F.fp6_code_to_fp16_bits(c6.astype(np.uint8)).view(np.float16)
    w6 = (v6.astype(np.float32) * s6.astype(np.float32)[None, :]).astype(np.float16)    # one rounding, as the reference's two hmuls
    return B, s, np.concatenate([w4, w6], axis=1)


@pytest.mark.parametrize("gs", [128, -1])
@pytest.mark.parametrize("m", [16, 32, 64, 128, 256, 512])
def test_every_code_in_every_position_through_the_gemm(m, gs):
    """One-hot rows of A make every output a single product: every instance of the kernel for up to 128 rows
    (m = 256: two launches of it) and the kernel for more rows (m = 512) must return the oracle's dequantised
    weights bit for bit."""
    dev = _dev()
    k, n4, n6 = 1024, 384, 128
    n = n4 + n6
    B, s, w_deq = _all_codes_problem(k, n4, n6, gs, seed=m + (0 if gs > 0 else 1))
    B, s = B.to(dev), s.to(dev)
    eye = torch.eye(k, dtype=torch.float16, device=dev)
    workspace = torch.zeros(64, dtype=torch.int32, device=dev)
    for r0 in range(0, k, m):
        a = eye[r0:r0 + m].contiguous()
        c = torch.zeros((m, n), dtype=torch.float16, device=dev)
        fm.mul(a, B, c, s, workspace, n6, group_size=gs, layout="b200")
        got = c.cpu().numpy()
        # exact equality of values (+0 and -0 compare equal)
        assert np.array_equal(got.astype(np.float32), w_deq[r0:r0 + m].astype(np.float32)), (m, gs, r0)
    assert fm.device_status(dev) == 0


def test_sweep_layer_every_m_against_the_oracle():
    """K = N = 8192, 256 FP6 columns, INT4 group 128: all M of the single-GPU sweep against the oracle."""
    dev = _dev()
    k = n = 8192
    qc, gs = 256, 128
    w = synth.make_weight_fp16(k, n, qc, seed=1)
    ww = fm.make_w46_weight(w, qc, gs, keep_dequantized=False, quant_device=dev)
    w_deq = _oracle_weight(w, qc, gs)
    for m in (1, 2, 4, 8, 16, 32, 64, 128):
        a = synth.make_activations(m, k, seed=m)
        c = _mul(a.to(dev), ww, m, n, qc, gs, dev).cpu().numpy().astype(np.float32)
        err = F.rel_frobenius(c, F.gemm_reference(a.numpy(), w_deq))
        assert err <= TOL, (m, err)


@pytest.mark.parametrize("k,n,qc,ms", [(4096, 22016, 256, (1, 16, 128)),      # Llama-2-7B gate_up
                                       (4096, 12288, 256, (1, 16)),           # Llama-2-7B qkv at small M
                                       (28672, 1024, 32, (1, 16, 128)),       # Llama-2-70B down, one of 8 shards
                                       (8192, 7168, 32, (16,))])              # Llama-2-70B gate_up, one of 8 shards
def test_llama_layers_against_the_oracle(k, n, qc, ms):
    dev = _dev()
    gs = 128
    w = synth.make_weight_fp16(k, n, qc, seed=k % 97)
    ww = fm.make_w46_weight(w, qc, gs, keep_dequantized=False, quant_device=dev)
    w_deq = _oracle_weight(w, qc, gs)
    for m in ms:
        a = synth.make_activations(m, k, seed=m + 1)
        c = _mul(a.to(dev), ww, m, n, qc, gs, dev).cpu().numpy().astype(np.float32)
        err = F.rel_frobenius(c, F.gemm_reference(a.numpy(), w_deq))
        assert err <= TOL, (k, n, m, err)

"""GPU parity of the fused epilogues (fp6m_mul_fused through fp6_marlin_b200.mul_fused): the gate / up
activation silu(gate) * up and the residual add, applied to the fp32 sums before the single rounding to fp16.
Checker: the oracle's dequantised weights (oracle/formats.py), an fp32-accumulated product and the same
epilogue in fp32 on the CPU.  Tolerance: relative Frobenius error <= 1e-3, as for the plain GEMM."""
import numpy as np
import pytest
import torch

import fp6_marlin_b200 as fm
from fp6_marlin_b200 import synth
from oracle import formats as F

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _oracle_weight(w: torch.Tensor, qc: int, gs: int) -> np.ndarray:
    k, n = w.shape
    nq = max(qc, 0)
    parts = []
    if n - nq:
        fn = (lambda x: F.int4_quantize_group(x, 128)) if gs > 0 else F.int4_quantize_per_channel
        parts.append(fn(w[:, : n - nq].numpy())[2])
    if nq:
        parts.append(F.fp6_codes_and_dequant(w[:, n - nq:].numpy())[2])
    return np.concatenate(parts, axis=1)


@pytest.mark.parametrize("m", [1, 16, 48, 200, 300])      # 200 rows: two launches of the kernel for up to 128 rows
@pytest.mark.parametrize("k,inter,qc,gs", [(1024, 1408, 256, 128), (512, 640, 64, -1), (2048, 512, 0, 128)])
def test_gate_up_activation_in_the_epilogue(m, k, inter, qc, gs):
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(k + inter + m)
    w_gate = (torch.randn((k, inter), generator=gen) * 0.02).half()
    w_up = (torch.randn((k, inter), generator=gen) * 0.02).half()
    w_gate[:, torch.randperm(inter, generator=gen)[: max(qc, 2) // 2]] *= 8.0     # outlier pairs
    weight, order = fm.make_gate_up_weight(w_gate, w_up, qc, gs)
    n = 2 * inter
    a = synth.make_activations(m, k, seed=m)
    c = torch.zeros((m, inter), dtype=torch.float16, device=dev)
    workspace = torch.zeros(max(n // 128 * 16, 64), dtype=torch.int32, device=dev)
    wd = weight.to(dev)
    fm.mul_fused(a.to(dev), wd.B, c, wd.s, workspace, qc if qc else -1, epilogue="silu_mul", group_size=gs)
    torch.cuda.synchronize()
    assert fm.device_status(dev) == 0
    # oracle: the interleaved matrix [g0 u0 g1 u1 ...] in the order the builder chose, INT4 pairs then FP6 pairs
    w_inter = torch.stack([w_gate[:, order], w_up[:, order]], dim=2).reshape(k, n).contiguous()
    full = F.gemm_reference(a.numpy(), _oracle_weight(w_inter, qc, gs))
    gate, up = full[:, 0::2], full[:, 1::2]
    ref = gate / (1.0 + np.exp(-gate)) * up
    err = F.rel_frobenius(c.cpu().numpy().astype(np.float32), ref)
    assert err <= TOL, (m, k, inter, qc, gs, err)


@pytest.mark.parametrize("m", [1, 16, 100, 200])
def test_residual_add_in_the_epilogue(m):
    dev = torch.device("cuda:0")
    k, n, qc, gs = 2048, 1024, 256, 128
    w = synth.make_weight_fp16(k, n, qc, seed=31)
    weight = fm.make_w46_weight(w, qc, gs, keep_dequantized=False).to(dev)
    a = synth.make_activations(m, k, seed=m)
    gen = torch.Generator().manual_seed(m)
    resid = torch.randn((m, n), generator=gen).half()
    workspace = torch.zeros(n // 128 * 16, dtype=torch.int32, device=dev)
    ref = F.gemm_reference(a.numpy(), _oracle_weight(w, qc, gs)) + resid.numpy().astype(np.float32)
    # into a separate output, and in place (C is the residual)
    c = torch.zeros((m, n), dtype=torch.float16, device=dev)
    fm.mul_fused(a.to(dev), weight.B, c, weight.s, workspace, qc, epilogue="residual", residual=resid.to(dev), group_size=gs)
    x = resid.to(dev).clone()
    fm.mul_fused(a.to(dev), weight.B, x, weight.s, workspace, qc, epilogue="residual", residual=x, group_size=gs)
    torch.cuda.synchronize()
    assert fm.device_status(dev) == 0
    for got in (c, x):
        err = F.rel_frobenius(got.cpu().numpy().astype(np.float32), ref)
        assert err <= TOL, (m, err)
    # one rounding: the fused result is at least as close to the fp32 reference as "GEMM, round, add, round"
    plain = torch.zeros((m, n), dtype=torch.float16, device=dev)
    fm.mul(a.to(dev), weight.B, plain, weight.s, workspace, qc, group_size=gs, layout="b200")
    two_roundings = (plain + resid.to(dev)).cpu().numpy().astype(np.float32)
    assert F.rel_frobenius(c.cpu().numpy().astype(np.float32), ref) <= F.rel_frobenius(two_roundings, ref) * 1.05


def test_fused_argument_errors():
    dev = torch.device("cuda:0")
    k, n = 256, 512
    weight = fm.make_w46_weight(synth.make_weight_fp16(k, n, -1), -1, 128, keep_dequantized=False).to(dev)
    a = synth.make_activations(4, k).to(dev)
    c = torch.zeros((4, n), dtype=torch.float16, device=dev)
    workspace = torch.zeros(64, dtype=torch.int32, device=dev)
    with pytest.raises(ValueError):
        fm.mul_fused(a, weight.B, c, weight.s, workspace, -1, epilogue="gelu", group_size=128)
    with pytest.raises(RuntimeError):
        fm.mul_fused(a, weight.B, c, weight.s, workspace, -1, epilogue="residual", residual=None, group_size=128)

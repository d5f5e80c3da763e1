"""Weight quantisers and the mixed INT4 / FP6 weight builder (torch ops + the C ABI).

The reference keeps this logic in its test script only: ``gen_int4_weight`` (test.py:85-121),
``gen_fp6_weight`` (test.py:13-58) and ``gen_mixed_weight`` (test.py:123-152).  The rules here are
the same rules (per-channel INT4 with scale ``max|w|*2/15``; FP6 with scale ``max|w|/28``, values
below 0.0625 flushed to zero, truncating cast), plus the group-128 INT4 rule the reference lacks
(``s = max|w_group|/7``, ``q = clamp(round(w/s), -8, 7) + 8``).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib
from ._lib import lib
from .api import encode_fp6_gpu, pack_b200, pack_b200_gpu

FP6_MAX = 28.0
FP6_MIN = 0.0625


def quantize_int4(w: torch.Tensor, group_size: int = -1):
    """fp16 W[k, n] -> (q uint8 [k, n] in 0..15, scales fp16, W_deq fp16 [k, n]).

    ``group_size=-1``: the reference's per-channel rule (test.py:87-98), scales of shape (n,).
    ``group_size=128``: symmetric groups along k, scales of shape (k/128, n).
    The dequantised weight is ``fp16(q - 8) * s`` with one fp16 multiply in both modes.
    """
    assert w.dtype == torch.float16 and w.dim() == 2
    k, n = w.shape
    if group_size <= 0:
        s = torch.max(torch.abs(w), 0, keepdim=True)[0]
        s = s * (2.0 / 15.0)
        q = torch.round(w / s).int() + 8
        q = torch.clamp(q, 0, 15)
        deq = (q - 8).half() * s
        return q.to(torch.uint8), s.reshape(n).contiguous(), deq
    assert group_size == 128 and k % group_size == 0
    wg = w.reshape(k // group_size, group_size, n)
    s = (torch.amax(torch.abs(wg), dim=1).float() / 7.0).half()
    s = torch.where(s == 0, torch.ones_like(s), s)
    q = torch.round(wg / s[:, None, :]).int()
    q = torch.clamp(q, -8, 7) + 8
    deq = ((q - 8).half() * s[:, None, :]).reshape(k, n)
    return q.reshape(k, n).to(torch.uint8), s.contiguous(), deq


def fake_quantize_fp6(w: torch.Tensor):
    """The FP6 pre-scaling of the reference's generator (test.py:19-27): returns (x, s) with
    ``x = w / s`` flushed below 0.0625 and clamped to +-28, ``s = max|w| / 28`` per column."""
    assert w.dtype == torch.float16 and w.dim() == 2
    s = torch.max(torch.abs(w), 0, keepdim=True)[0]
    s = s * (1.0 / FP6_MAX)
    x = w / s
    x = torch.where(torch.abs(x) < FP6_MIN, torch.zeros_like(x), x)
    x = torch.clamp(x, -FP6_MAX, FP6_MAX)
    return x, s.reshape(-1).contiguous()


def encode_fp6(x: torch.Tensor) -> torch.Tensor:
    """fp16 values in the FP6 range -> codes ``s eee mm`` (uint8), truncating (weight_quant.cpp:27-91)."""
    if x.dtype != torch.float16:
        raise ValueError("Input tensor should be of type float16.")
    src = x.detach().cpu().contiguous()
    codes = torch.empty(src.shape, dtype=torch.uint8)
    rc = lib.fp6m_encode_fp6(src.data_ptr(), codes.data_ptr(), src.numel())
    if rc == _lib.ERR_VALUE_RANGE:
        raise ValueError("Input value out of range for FP6.")
    if rc:
        raise RuntimeError(f"fp6m_encode_fp6 failed with code {rc}")
    return codes


def decode_fp6(codes: torch.Tensor) -> torch.Tensor:
    """Codes -> their exact E3M2 values as fp16 (weight_prepacking.cpp:199-212 with unit scale)."""
    c = codes.to(torch.int32)
    sign = torch.where((c & 0x20) != 0, -1.0, 1.0)
    e = (c >> 2) & 7
    m = (c & 3).float()
    normal = torch.pow(2.0, (e - 3).float()) * (1.0 + m / 4.0)
    sub = m / 16.0
    return (sign * torch.where(e > 0, normal, sub)).half()


def quantize_fp6(w: torch.Tensor):
    """fp16 W[k, n] -> (codes uint8 [k, n], scales fp16 (n,), W_deq fp16 [k, n]); W_deq is the exact
    code value times the column scale with one fp16 multiply, as ``dequantize`` returns it."""
    x, s = fake_quantize_fp6(w)
    codes = encode_fp6_gpu(x) if x.device.type == "cuda" else encode_fp6(x)
    deq = decode_fp6(codes) * s.reshape(1, -1)
    return codes, s, deq


@dataclass
class W46Weight:
    """A mixed-precision weight in the b200 layout: columns ``[INT4 | FP6]``."""
    B: torch.Tensor            # packed words, int32, flat
    s: torch.Tensor            # scales, fp16, flat (b200 order)
    k: int
    n: int
    quant_cols: int            # number of FP6 columns (-1 = none)
    group_size: int            # 128 or -1
    w_deq: torch.Tensor | None = None   # (k, n) fp16 dequantised weights, if kept

    def to(self, device):
        return W46Weight(self.B.to(device), self.s.to(device), self.k, self.n, self.quant_cols,
                         self.group_size, None if self.w_deq is None else self.w_deq.to(device))


def make_w46_weight(w: torch.Tensor, quant_cols: int = -1, group_size: int = 128, keep_dequantized: bool = True,
                    quant_device=None) -> W46Weight:
    """Quantise and pack fp16 W[k, n] whose last ``quant_cols`` columns are to be FP6 and the rest
    INT4 - the counterpart of ``gen_mixed_weight`` (test.py:123-152) for the b200 layout.
    With ``quant_device`` (a CUDA device) everything - the INT4 rule, the FP6 scaling and truncating
    cast, the packing - runs on that GPU (same IEEE fp16 arithmetic, same bytes) and the weight stays
    there; without it the weight is prepared and kept on the CPU."""
    k, n = w.shape
    qc = max(quant_cols, 0)
    w4, w6 = w[:, : n - qc], w[:, n - qc:]
    q4 = s4 = d4 = c6 = s6 = d6 = None
    on_gpu = quant_device is not None and torch.device(quant_device).type == "cuda"
    if n - qc > 0:
        src = w4.contiguous() if quant_device is None else w4.to(quant_device).contiguous()
        q4, s4, d4 = quantize_int4(src, group_size)
        if not keep_dequantized:
            d4 = None
    if qc > 0:
        src = w6.contiguous() if quant_device is None else w6.to(quant_device).contiguous()
        c6, s6, d6 = quantize_fp6(src)
        if not keep_dequantized:
            d6 = None
    B, s = (pack_b200_gpu if on_gpu else pack_b200)(q4, c6, s4, s6, k, n, quant_cols, group_size)
    deq = None
    if keep_dequantized:
        deq = torch.cat([d for d in (d4, d6) if d is not None], dim=1).contiguous()
    return W46Weight(B, s, k, n, quant_cols, group_size, deq)


def select_outlier_columns(w: torch.Tensor, quant_cols: int) -> torch.Tensor:
    """Column permutation that moves the ``quant_cols`` columns of largest abs-max to the end
    (ties broken toward the lower index) and keeps the order of the others."""
    n = w.shape[1]
    amax = torch.amax(torch.abs(w.float()), dim=0)
    order = torch.sort(amax, descending=True, stable=True)[1]
    outliers = torch.sort(order[:quant_cols])[0]
    mask = torch.ones(n, dtype=torch.bool, device=w.device)
    mask[outliers] = False
    return torch.cat([torch.arange(n, device=w.device)[mask], outliers])


def make_gate_up_weight(w_gate: torch.Tensor, w_up: torch.Tensor, quant_cols: int = 256, group_size: int = 128,
                        keep_dequantized: bool = False, quant_device=None):
    """Gate and up projections W_gate[k, i], W_up[k, i] (fp16) -> one packed weight of 2i columns for
    ``mul_fused(..., epilogue="silu_mul")``, plus the order of the outputs.

    Pairs stay together: the ``quant_cols / 2`` pairs (gate_j, up_j) whose larger abs-max is largest become
    FP6 (ties toward the lower j), the others INT4; inside each region the columns alternate gate_j, up_j, in
    increasing j.  Returns ``(weight, order)`` where output column t of the fused GEMM is
    ``silu(x @ W_gate[:, order[t]]) * (x @ W_up[:, order[t]])``.
    """
    assert w_gate.shape == w_up.shape and w_gate.dtype == torch.float16 and w_up.dtype == torch.float16
    k, inter = w_gate.shape
    qc = max(quant_cols, 0)
    assert qc % 2 == 0 and qc // 2 <= inter
    score = torch.maximum(torch.amax(torch.abs(w_gate.float()), dim=0), torch.amax(torch.abs(w_up.float()), dim=0))
    ranked = torch.sort(score, descending=True, stable=True)[1]
    outliers = torch.sort(ranked[: qc // 2])[0]
    mask = torch.ones(inter, dtype=torch.bool, device=w_gate.device)
    mask[outliers] = False
    order = torch.cat([torch.arange(inter, device=w_gate.device)[mask], outliers])
    w = torch.stack([w_gate[:, order], w_up[:, order]], dim=2).reshape(k, 2 * inter).contiguous()
    weight = make_w46_weight(w, quant_cols if qc else -1, group_size, keep_dequantized, quant_device)
    return weight, order

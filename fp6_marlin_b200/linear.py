"""A linear layer on top of ``mul``: picks the FP6 columns, packs, runs, puts the outputs back in order.

The reference leaves the column order to its caller: ``mul`` returns the output features as
``[INT4 columns | FP6 columns]`` (an attempt to undo that inside the binding is commented out,
fp6_marlin/fp6_marlin_cuda.cpp:93-122).  This module owns that bookkeeping: the ``quant_cols`` output
features with the largest magnitude become the FP6 columns, the permutation is remembered, and
``forward`` either restores the model's feature order or hands the permuted result on together
with ``output_permutation`` so that the next layer can fold it into its input features.
"""
from __future__ import annotations

import torch

from . import api
from .quant import W46Weight, make_w46_weight, select_outlier_columns


class W46Linear(torch.nn.Module):
    """``y = x @ W.T (+ bias)`` with W (out_features, in_features) quantised to mixed INT4 / FP6-E3M2.

    ``quant_cols`` output features (-1 / 0: none; the rest stay INT4) are kept in FP6; ``group_size`` is 128
    (INT4 scales per 128 input features) or -1 (one scale per output feature, the reference's rule).
    """

    def __init__(self, weight: torch.Tensor, quant_cols: int = 256, group_size: int = 128, bias: torch.Tensor | None = None,
                 restore_order: bool = True, quant_device=None):
        super().__init__()
        if weight.dim() != 2:
            raise ValueError("weight must be (out_features, in_features)")
        self.out_features, self.in_features = weight.shape
        self.quant_cols = quant_cols if quant_cols and quant_cols > 0 else -1
        self.group_size = group_size
        self.restore_order = restore_order
        w_kn = weight.detach().to(torch.float16).t().contiguous().cpu()          # (k, n): columns = output features
        qc = max(self.quant_cols, 0)
        perm = select_outlier_columns(w_kn, qc) if qc else torch.arange(self.out_features)
        packed: W46Weight = make_w46_weight(w_kn[:, perm].contiguous(), self.quant_cols, group_size,
                                            keep_dequantized=False, quant_device=quant_device)
        inverse = torch.empty_like(perm)
        inverse[perm] = torch.arange(self.out_features)
        self.register_buffer("B", packed.B)
        self.register_buffer("s", packed.s)
        self.register_buffer("output_permutation", perm)       # column j of mul's output is feature perm[j]
        self.register_buffer("inverse_permutation", inverse)   # feature f is column inverse[f] of mul's output
        self.register_buffer("workspace", torch.zeros(max(self.out_features // 128 * 16, 64), dtype=torch.int32))
        self.register_buffer("bias", None if bias is None else bias.detach().to(torch.float16).clone())

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.dtype != torch.float16:
            raise ValueError("activations must be float16")
        lead = x.shape[:-1]
        a = x.reshape(-1, self.in_features).contiguous()
        c = torch.empty((a.shape[0], self.out_features), dtype=torch.float16, device=a.device)
        api.mul(a, self.B, c, self.s, self.workspace, self.quant_cols, group_size=self.group_size, layout="b200")
        if self.restore_order:
            c = c.index_select(1, self.inverse_permutation)
            if self.bias is not None:
                c = c + self.bias
        elif self.bias is not None:
            c = c + self.bias.index_select(0, self.output_permutation)
        return c.reshape(*lead, self.out_features)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, fp6_columns={max(self.quant_cols, 0)}, "
                f"group_size={self.group_size}, restore_order={self.restore_order}")

"""N-sharding of a mixed INT4 / FP6 layer over the GPUs of one node, and the exchange step.

The reference has no multi-GPU code.  Output columns are independent, so a layer is split along N:
rank r of g keeps INT4 columns [r*n4/g, (r+1)*n4/g) and FP6 columns [r*qc/g, (r+1)*qc/g) of the
``[INT4 | FP6]``-ordered matrix, packed as its own ``[INT4 | FP6]`` problem, every rank holds all of
A, and the one exchange step is an all-gather of the (M, N/g) output blocks.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class ShardPlan:
    n: int
    quant_cols: int        # FP6 columns of the whole layer (0 = none)
    world: int

    @property
    def n4(self) -> int:
        return self.n - self.quant_cols

    @property
    def n_local(self) -> int:
        return self.n // self.world

    @property
    def qc_local(self) -> int:
        return self.quant_cols // self.world

    def check(self) -> None:
        if self.n4 % self.world or self.quant_cols % self.world:
            raise ValueError("both column regions must divide evenly over the ranks")
        if (self.n4 // self.world) % 8 or self.qc_local % 8:
            raise ValueError("every shard needs multiples of 8 columns per region")

    def local_columns(self, rank: int) -> torch.Tensor:
        """Global column indices held by `rank`, in the order of its local matrix."""
        a, b = self.n4 // self.world, self.qc_local
        return torch.cat([torch.arange(rank * a, (rank + 1) * a),
                          self.n4 + torch.arange(rank * b, (rank + 1) * b)])

    def gather_index(self) -> torch.Tensor:
        """Permutation p: position i of the rank-major concatenation of the shards holds global
        column p[i]."""
        return torch.cat([self.local_columns(r) for r in range(self.world)])


def shard_weight(w: torch.Tensor, plan: ShardPlan, rank: int) -> torch.Tensor:
    """Columns of fp16 W[k, n] (already ordered [INT4 | FP6]) that belong to `rank`."""
    plan.check()
    return w[:, plan.local_columns(rank)].contiguous()


def assemble(gathered: torch.Tensor, plan: ShardPlan) -> torch.Tensor:
    """(g, M, N/g) all-gather result -> (M, N) in the layer's global column order."""
    g, m, n_local = gathered.shape
    assert g == plan.world and n_local == plan.n_local
    flat = gathered.permute(1, 0, 2).reshape(m, g * n_local)
    out = torch.empty((m, plan.n), dtype=gathered.dtype, device=gathered.device)
    out[:, plan.gather_index().to(gathered.device)] = flat
    return out


def all_gather_columns(c_local: torch.Tensor, out: torch.Tensor | None = None, group=None) -> torch.Tensor:
    """The exchange step: every rank contributes its (M, N/g) block; returns (g, M, N/g)."""
    world = dist.get_world_size(group)
    if out is None:
        out = torch.empty((world,) + tuple(c_local.shape), dtype=c_local.dtype, device=c_local.device)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(out, c_local.contiguous(), group=group)
    else:   # CPU ranks (gloo): the list form
        dist.all_gather([out[r] for r in range(world)], c_local.contiguous(), group=group)
    return out


class ShardedW46Linear:
    """One rank's part of an N-sharded W(4&6)A16 layer: local GEMM + all-gather of the columns."""

    def __init__(self, w_fp16: torch.Tensor, quant_cols: int, group_size: int, rank: int, world: int, device):
        from .quant import make_w46_weight
        self.plan = ShardPlan(w_fp16.shape[1], max(quant_cols, 0), world)
        self.plan.check()
        self.rank, self.device = rank, torch.device(device)
        local = shard_weight(w_fp16, self.plan, rank)
        qc_local = self.plan.qc_local if quant_cols > 0 else -1
        self.weight = make_w46_weight(local, qc_local, group_size, keep_dequantized=False,
                                      quant_device=self.device).to(self.device)
        self.workspace = torch.zeros(max(self.plan.n_local // 128 * 16, 64), dtype=torch.int32, device=self.device)

    def forward_local(self, a: torch.Tensor, c_local: torch.Tensor | None = None) -> torch.Tensor:
        from .api import mul
        if c_local is None:
            c_local = torch.empty((a.shape[0], self.plan.n_local), dtype=torch.float16, device=self.device)
        mul(a, self.weight.B, c_local, self.weight.s, self.workspace, self.weight.quant_cols,
            group_size=self.weight.group_size, layout="b200")
        return c_local

    def forward(self, a: torch.Tensor) -> torch.Tensor:
        """(M, K) activations (replicated) -> (g, M, N/g) gathered output; `assemble` orders the columns."""
        return all_gather_columns(self.forward_local(a))

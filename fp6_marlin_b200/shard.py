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


class _DevicePointer:
    """Lets torch wrap raw device memory (``torch.as_tensor`` reads ``__cuda_array_interface__``)."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 2}


class PeerExchange:
    """Fused exchange step: every rank's GEMM stores its output columns straight into the full-width output
    buffers of ALL ranks (peer memory over NVLink, mapped with CUDA IPC), in the layer's global column order,
    and a signal / bounded-wait pair of tiny kernels stands in for the collective.

    ``outputs`` are double-buffered: step t uses buffer t % 2, so a rank that already runs step t + 1 does
    not overwrite what a slower rank still reads from step t.  Set-up allocates and exchanges IPC handles
    through ``torch.distributed`` (object all-gather); the hot path (``mul_scatter`` + ``finish``) makes no
    collective call and is CUDA-graph capturable.
    """

    def __init__(self, plan: ShardPlan, rank: int, m_max: int, device, group=None):
        import ctypes

        from ._lib import lib
        self._lib, self._ct = lib, ctypes
        self.plan, self.rank, self.world = plan, rank, plan.world
        self.device = torch.device(device)
        self.dev_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.m_max = m_max
        self.step = 0
        out_bytes = 2 * m_max * plan.n * 2
        flag_bytes = 256
        self._own = []          # (ptr, handle) of this rank's buffers: outputs, flags
        for nbytes in (out_bytes, flag_bytes):
            ptr = ctypes.c_void_p()
            handle = ctypes.create_string_buffer(64)
            rc = lib.fp6m_peer_alloc(nbytes, self.dev_index, ctypes.byref(ptr), handle)
            if rc:
                raise RuntimeError(f"fp6m_peer_alloc failed with code {rc}")
            self._own.append((ptr.value, handle.raw))
        handles = [None] * self.world
        dist.all_gather_object(handles, [h for _, h in self._own], group=group)
        self._opened = []
        self.out_ptrs, self.flag_ptrs = [], []
        for r in range(self.world):
            if r == rank:
                self.out_ptrs.append(self._own[0][0])
                self.flag_ptrs.append(self._own[1][0])
                continue
            ptrs = []
            for h in handles[r]:
                ptr = ctypes.c_void_p()
                rc = lib.fp6m_peer_open(ctypes.create_string_buffer(h, 64), self.dev_index, ctypes.byref(ptr))
                if rc:
                    raise RuntimeError(f"fp6m_peer_open failed with code {rc} (rank {r})")
                ptrs.append(ptr.value)
                self._opened.append(ptr.value)
            self.out_ptrs.append(ptrs[0])
            self.flag_ptrs.append(ptrs[1])
        # this rank's own memory as tensors
        self.outputs = torch.as_tensor(_DevicePointer(self._own[0][0], (2, m_max, plan.n), "<f2"), device=self.device)
        self._step_dev = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._flag_table = (ctypes.c_void_p * self.world)(*self.flag_ptrs)
        self._out_tables = [(ctypes.c_void_p * self.world)(*[p + b * m_max * plan.n * 2 for p in self.out_ptrs]) for b in (0, 1)]
        dist.barrier(group=group)      # every rank has mapped every buffer before anyone stores

    def mul_scatter(self, a, weight, workspace, buffer: int):
        """Local GEMM of this rank's shard; results go to buffer ``buffer`` (0/1) of every rank."""
        from . import _lib
        from .api import _device_buffers, _ptr
        m, k = a.shape
        if m > self.m_max:
            raise ValueError("mul_scatter: more rows than the exchange was built for")
        plan = self.plan
        _, scratch, status = _device_buffers(self.device, (m, plan.n_local, k, weight.quant_cols))
        stream = torch.cuda.current_stream(self.device).cuda_stream
        col4 = self.rank * (plan.n4 // plan.world)
        col6 = plan.n4 + self.rank * plan.qc_local
        rc = self._lib.fp6m_mul_scatter(_ptr(a), _ptr(weight.B), self._out_tables[buffer], self.world, plan.n, col4, col6,
                                        _ptr(weight.s), m, plan.n_local, k, _ptr(workspace),
                                        workspace.numel() * workspace.element_size(), _ptr(scratch), scratch.numel(),
                                        self.dev_index, stream, -1, -1, -1, 16, weight.quant_cols, weight.group_size,
                                        _lib.LAYOUT_B200, _ptr(status))
        if rc:
            raise RuntimeError(f"fp6m_mul_scatter failed with code {rc}: {_lib.last_cuda_error()}")

    def finish(self):
        """Signal "my shard has landed everywhere" and hold the stream until every rank has signalled."""
        from .api import _device_buffers, _ptr
        _, _, status = _device_buffers(self.device)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = self._lib.fp6m_peer_signal_wait(self._flag_table, self.world, self.rank, _ptr(self._step_dev), _ptr(status),
                                             self.dev_index, stream)
        if rc:
            raise RuntimeError(f"peer signal/wait failed with code {rc}")

    def close(self):
        """Unmaps the peers' buffers and frees this rank's; call on every rank after a barrier."""
        for ptr in self._opened:
            self._lib.fp6m_peer_close(ptr, self.dev_index)
        self._opened = []
        self.outputs = None
        for ptr, _ in self._own:
            self._lib.fp6m_peer_free(ptr, self.dev_index)
        self._own = []

"""Host logic of the N-sharded layer, on CPU ranks (gloo, world size 2): the column plan, the
all-gather of output columns and the re-assembly reproduce the unsharded product bit for bit."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fp6_marlin_b200 import shard


def test_plan_columns_partition_the_layer():
    for n, qc, world in [(8192, 256, 8), (10240, 256, 8), (1024, 0, 2), (57344, 256, 4)]:
        plan = shard.ShardPlan(n, qc, world)
        plan.check()
        idx = plan.gather_index()
        assert idx.numel() == n and torch.equal(torch.sort(idx)[0], torch.arange(n))
        cols = plan.local_columns(world - 1)
        assert cols.numel() == n // world
        assert int(cols[-1]) == n - 1 if qc else True
    with pytest.raises(ValueError):
        shard.ShardPlan(1000, 250, 8).check()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        m, k, n, qc = 5, 64, 512, 128
        w = torch.randn(k, n).half()
        a = torch.randn(m, k).half()
        plan = shard.ShardPlan(n, qc, world)
        w_local = shard.shard_weight(w, plan, rank)
        c_local = (a.float() @ w_local.float()).half()          # stands in for the local GEMM
        gathered = shard.all_gather_columns(c_local)
        full = shard.assemble(gathered, plan)
        expect = (a.float() @ w.float()).half()
        ret[rank] = bool(torch.equal(full, expect))
    finally:
        dist.destroy_process_group()


def test_all_gather_and_assembly_on_two_cpu_ranks():
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}

#!/usr/bin/env python
"""Benchmark of the W(4&6)A16 GEMM path.

Workload (one "step" = one `mul` call): the square layer of the single-GPU sweep, K = N = 8192,
M = 16 rows of fp16 activations, 256 FP6 columns + INT4 group-128 elsewhere, seeded synthetic
values (fp6_marlin_b200/synth.py).  The metric is effective HBM bandwidth: algorithmic bytes of
one GEMM (A + packed weights + scales + C, the form of the reference's bench.py:46-50) divided by
its latency.

  value      K steps replayed from CUDA graphs (the launch-bound inner loop is captured), inputs
             resident in HBM, each step on a different one of several weight copies so that the
             working set exceeds L2; timed with CUDA events on the launching stream.
  e2e        the same K steps through the public Python API with HOST buffers: every step copies A
             from pinned host memory, calls mul, and copies C back to pinned host memory.
  roofline   achieved GB/s of the GEMM kernel in the timed region against the measured HBM peak
             (MEASURED_PEAKS.json), `traffic` from an ncu capture (profiles/).
  cpu_baseline / --impl reference
             the reference's CPU path for the same layer - FP6 columns dequantised by the
             reference's own host code (oracle/_ref), INT4 columns by the rule of its test script
             ((q-8).half()*s), then torch.matmul in fp32 - timed on the host cores.

With N > 1 GPUs (torchrun) the layer's output columns are sharded over the ranks and every step
ends with an NCCL all-gather of the output columns: total work is fixed ("strong" scaling).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

K_DIM, N_DIM, M_ROWS, QUANT_COLS, GROUP = 8192, 8192, 16, 256, 128
METRIC = "W4&6A16 GEMM effective HBM bandwidth (K=N=8192, M=16, 256 FP6 cols, INT4 g128)"
UNIT = "GB/s"
GRAPH_CHUNK = 500
WEIGHT_COPIES = 8          # 8 x 35 MB of packed weights > 2 x the 126 MB L2


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20000)
    ap.add_argument("--warmup", type=int, default=200)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--sweep", action="store_true", help="also time the other M values and layer shapes")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: all-gather of the output columns fused into the GEMM epilogue as peer stores, or NCCL")
    ap.add_argument("--only-shape", default=None, metavar="K,N,M",
                    help="time just this shape the way --sweep does and print its record (used for profiling other shapes)")
    ap.add_argument("--no-overlap", action="store_true",
                    help="launch the GEMMs without programmatic dependent launch (no overlap of consecutive steps)")
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi in loop mode beside the timed regions (reads settings only)."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_uuid: str | None):
        self.rows = []
        self.proc = None
        cmd = ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"]
        if gpu_uuid:
            cmd += ["-i", gpu_uuid if gpu_uuid.startswith("GPU-") else "GPU-" + gpu_uuid]
        try:
            self.proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 9:
                self.rows.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, sm_max, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                sm_max.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # "under load": samples in the upper half of what was seen (idle samples sit at low clocks)
        load = [x for x in sm if x >= 0.5 * max(sm)] if sm else []
        return {"sm_mhz": statistics.median(load) if load else None,
                "sm_max_mhz": max(sm_max) if sm_max else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------
# the reference's CPU path (checker code: the one place bench.py executes oracle/)
# ------------------------------------------------------------------------------------------------
def cpu_reference_step_fn(n_int4_cols: int):
    """Returns (step(), algorithmic_bytes, description) for the reference's CPU path on a column slab
    of the benchmark layer: `n_int4_cols` INT4 columns plus all 256 FP6 columns."""
    import numpy as np
    import torch

    from fp6_marlin_b200 import synth
    from fp6_marlin_b200.quant import fake_quantize_fp6, quantize_int4
    from oracle import ref_lib

    n = n_int4_cols + QUANT_COLS
    w = synth.make_weight_fp16(K_DIM, N_DIM, QUANT_COLS, seed=0)
    w = torch.cat([w[:, :n_int4_cols], w[:, N_DIM - QUANT_COLS:]], dim=1).contiguous()
    a = synth.make_activations(M_ROWS, K_DIM)
    q4, s4, _ = quantize_int4(w[:, :n_int4_cols].contiguous(), GROUP)
    x6, s6 = fake_quantize_fp6(w[:, n_int4_cols:].contiguous())
    use_ref = ref_lib.available()
    if use_ref:
        # one-off weight preparation, timed for the record: quantize + prepacking of the FP6 columns
        t0 = time.perf_counter()
        stream = ref_lib.quantize(np.ascontiguousarray(x6.t().numpy()).reshape(K_DIM, QUANT_COLS))
        ref_lib.prepacking(stream)
        prep_s = time.perf_counter() - t0
        s6_np = s6.numpy()
    else:
        from oracle import formats
        t0 = time.perf_counter()
        stream = formats.fp6_quantize(np.ascontiguousarray(x6.t().numpy()).reshape(K_DIM, QUANT_COLS))
        prep_s = time.perf_counter() - t0
        s6_np = s6.numpy()

    def step():
        # dequantise (test.py:98 rule for INT4; dequantMatrix_fp6_to_fp16 for FP6), then fp32 matmul
        w4 = ((q4.to(torch.int32) - 8).half().reshape(K_DIM // GROUP, GROUP, n_int4_cols) * s4[:, None, :]).reshape(K_DIM, n_int4_cols)
        if use_ref:
            w6 = torch.from_numpy(ref_lib.dequantize(stream, s6_np)).t()
        else:
            w6 = torch.from_numpy(formats.fp6_dequant(stream, s6_np)).t()
        w_deq = torch.cat([w4, w6], dim=1)
        return torch.matmul(a.float(), w_deq.float())

    nbytes = synth.algorithmic_bytes(M_ROWS, K_DIM, n, QUANT_COLS, GROUP)
    kind = "reference" if use_ref else "port"
    desc = (f"dequantize+fp32 matmul of a {K_DIM}x{n} column slab ({n_int4_cols} INT4 g128 cols + {QUANT_COLS} FP6 cols) "
            f"of the K=N=8192 layer, M=16; one-off FP6 quantize+prepack of the slab took {prep_s * 1e3:.0f} ms")
    return step, nbytes, kind, desc


def time_cpu_reference(steps: int, warmup: int, budget_s: float):
    """Times the reference's CPU path; sizes the column slab so that the run stays within budget."""
    import torch
    n4_full = N_DIM - QUANT_COLS
    n4 = n4_full
    step, nbytes, kind, desc = cpu_reference_step_fn(n4)
    t0 = time.perf_counter()
    step()
    one = time.perf_counter() - t0
    total = max(steps + warmup, 1)
    while one * total > budget_s and n4 > 256:
        n4 = max(256, (int(n4 * budget_s / (one * total)) // 128) * 128)
        step, nbytes, kind, desc = cpu_reference_step_fn(n4)
        t0 = time.perf_counter()
        step()
        one = time.perf_counter() - t0
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    elapsed = time.perf_counter() - t0
    ms = elapsed / max(steps, 1) * 1e3
    return {"value": nbytes / (ms * 1e-3) / 1e9, "unit": UNIT, "cores": torch.get_num_threads(),
            "kind": kind, "sample": desc, "ms_per_step": ms, "host_cpus": os.cpu_count()}


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    res = time_cpu_reference(args.steps, args.warmup, budget_s=150.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp16 weights dequantised on the host, fp32 matmul",
        "data": "synthetic", "config": {"workload": "cfg1 square layer K=N=8192 M=16 qc=256 INT4-g128 (CPU path of the reference)"},
        "cpu_baseline": {"value": res["value"], "unit": UNIT, "cores": res["cores"], "kind": res["kind"], "sample": res["sample"]},
        "e2e": {"value": res["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# the B200 arm
# ------------------------------------------------------------------------------------------------
def b200_arm(args):
    import torch
    import torch.distributed as dist

    import fp6_marlin_b200 as fm
    from fp6_marlin_b200 import shard, synth

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA GPU (no CPU fallback)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if args.only_shape:
        k, n, m = (int(x) for x in args.only_shape.split(","))
        fm.set_launch_overlap(not args.no_overlap)
        print(json.dumps(run_sweep(fm, synth, dev, measured_peaks(), only=(k, n, m))[0]))
        return
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    assert world == args.gpus or world == 1, "launch with torchrun --nproc-per-node == --gpus"

    n_local, qc_local = N_DIM // world, QUANT_COLS // world
    w = synth.make_weight_fp16(K_DIM, N_DIM, QUANT_COLS, seed=0)
    if world > 1:
        w = shard.shard_weight(w, shard.ShardPlan(N_DIM, QUANT_COLS, world), rank)
    weight = fm.make_w46_weight(w, qc_local, GROUP, keep_dequantized=False, quant_device=dev)
    n_copies = max(WEIGHT_COPIES, int(280e6 // (weight.B.numel() * 4)) + 1)      # > 2 x L2 in total
    copies = [(weight.B.to(dev).clone(), weight.s.to(dev).clone()) for _ in range(n_copies)]
    a_host = synth.make_activations(M_ROWS, K_DIM).pin_memory()
    a_dev = a_host.to(dev)
    c_dev = torch.zeros((M_ROWS, n_local), dtype=torch.float16, device=dev)
    gathered = torch.zeros((world, M_ROWS, n_local), dtype=torch.float16, device=dev) if world > 1 else None
    c_host = torch.zeros((world, M_ROWS, n_local), dtype=torch.float16).pin_memory()
    workspace = torch.zeros(max(n_local // 128 * 16, 64), dtype=torch.int32, device=dev)
    stream = torch.cuda.Stream(device=dev)
    # consecutive GEMMs of a decode step: each may set itself up and prefetch its (static) weights while
    # the previous kernel of the stream drains; activations, outputs and scratch wait for that kernel
    fm.set_launch_overlap(not args.no_overlap)

    exchange = None
    if world > 1 and args.exchange == "peer":
        from types import SimpleNamespace
        exchange = shard.PeerExchange(shard.ShardPlan(N_DIM, QUANT_COLS, world), rank, M_ROWS, dev)
        shards = [SimpleNamespace(B=B, s=s, quant_cols=qc_local, group_size=GROUP) for B, s in copies]

    def step(i, a):
        if exchange is not None:
            # every rank stores its columns into every rank's (M, N) output; signal + bounded wait complete the step
            exchange.mul_scatter(a, shards[i % n_copies], workspace, i % 2)
            exchange.finish()
            return
        B, s = copies[i % n_copies]
        fm.mul(a, B, c_dev, s, workspace, qc_local, group_size=GROUP, layout="b200")
        if world > 1:
            dist.all_gather_into_tensor(gathered, c_dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(str(torch.cuda.get_device_properties(dev).uuid) if rank == 0 else None) if rank == 0 else None

    exchange_ok = None
    with torch.cuda.stream(stream):
        for i in range(max(args.warmup, 3)):
            step(i, a_dev)
        torch.cuda.synchronize()
        if exchange is not None:
            # parity of the fused exchange: the same step through the NCCL all-gather + column assembly
            last = max(args.warmup, 3) - 1
            B, s = copies[last % n_copies]
            fm.mul(a_dev, B, c_dev, s, workspace, qc_local, group_size=GROUP, layout="b200")
            dist.all_gather_into_tensor(gathered, c_dev)
            expect = shard.assemble(gathered, shard.ShardPlan(N_DIM, QUANT_COLS, world))
            torch.cuda.synchronize()
            ok = torch.tensor([int(torch.equal(expect, exchange.outputs[last % 2]))], device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            exchange_ok = bool(ok.item())

        # ---- value: K steps, captured in CUDA graphs when single-GPU
        chunk = min(GRAPH_CHUNK, args.steps)
        graphs = []
        if True:
            for count in ([chunk] if args.steps % chunk == 0 else [chunk, args.steps % chunk]):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    for i in range(count):
                        step(i, a_dev)
                graphs.append((g, count))
            graphs[0][0].replay()
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        for _ in range(args.steps // chunk):
            graphs[0][0].replay()
        if args.steps % chunk:
            graphs[1][0].replay()
        ev1.record(stream)
        barrier()
        ms_total = ev0.elapsed_time(ev1)

        # ---- e2e: host buffers, copies inside the timed region
        e2e_steps = args.steps
        for i in range(3):
            a_dev.copy_(a_host, non_blocking=True)
            step(i, a_dev)
            c_host[0].copy_(c_dev, non_blocking=True)
        barrier()
        ev2, ev3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev2.record(stream)
        for i in range(e2e_steps):
            a_dev.copy_(a_host, non_blocking=True)
            step(i, a_dev)
            if exchange is not None:
                c_host.view(M_ROWS, N_DIM).copy_(exchange.outputs[i % 2], non_blocking=True)
            elif world > 1:
                c_host.copy_(gathered, non_blocking=True)
            else:
                c_host[0].copy_(c_dev, non_blocking=True)
        ev3.record(stream)
        barrier()
        ms_e2e_total = ev2.elapsed_time(ev3)

    clocks = sampler.stop() if sampler else None
    status = fm.device_status(dev)

    if world > 1:
        t = torch.tensor([ms_total, ms_e2e_total], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, ms_e2e_total = t.tolist()

    nbytes = synth.algorithmic_bytes(M_ROWS, K_DIM, N_DIM, QUANT_COLS, GROUP)          # whole layer
    nbytes_local = synth.algorithmic_bytes(M_ROWS, K_DIM, n_local, qc_local, GROUP)     # one rank's kernel
    ms_step = ms_total / args.steps
    ms_e2e = ms_e2e_total / e2e_steps
    peaks = measured_peaks()
    value = nbytes / (ms_step * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp16 (fp32 accumulate)",
        "data": "synthetic",
        "config": {"workload": "cfg1 square layer K=N=8192 M=16 qc=256 INT4-g128", "M": M_ROWS, "K": K_DIM, "N": N_DIM,
                   "quant_cols": QUANT_COLS, "group_size": GROUP,
                   "l2": f"{n_copies} rotating weight copies ({n_copies * weight.B.numel() * 4 / 1e6:.0f} MB) exceed L2",
                   "parallelism": "single GPU" if world == 1 else (
                       f"N-sharded over {world} GPUs, output columns exchanged by peer stores in the GEMM epilogue + signal/wait kernels"
                       if exchange is not None else f"N-sharded over {world} GPUs + NCCL all-gather of output columns"),
                   "graph": True, "launch_overlap": not args.no_overlap},
        "e2e": {"value": nbytes / (ms_e2e * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": a_host.numel() * 2, "d2h_bytes_per_step": M_ROWS * N_DIM * 2},
        "gpu_launches": args.steps * (2 if exchange is not None else 1),
        "clocks": clocks,
        "device_status": status,
    }
    if exchange_ok is not None:
        line["config"]["exchange_matches_nccl_all_gather"] = exchange_ok
    if world == 1:
        achieved = nbytes_local / (ms_step * 1e-3) / 1e9
        line["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                            "frac": achieved / peaks["hbm_gbs"], "peak_source": f"of {peaks['source']}",
                            "algorithmic_bytes": nbytes_local, "traffic": read_traffic_from_profile()}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cb = time_cpu_reference(steps=5, warmup=1, budget_s=25.0)
        line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
    if args.sweep and world == 1:
        line["sweep"] = run_sweep(fm, synth, dev, peaks)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        # CUDA graphs that captured NCCL work must go before the communicator does; a watchdog ends the
        # process if the tear-down of the process group stalls (the result line is already printed)
        graphs.clear()
        torch.cuda.synchronize()
        sys.stdout.flush()
        threading.Timer(20.0, lambda: os._exit(0)).start()
        dist.barrier()
        if exchange is not None:
            exchange.close()
            dist.barrier()
        dist.destroy_process_group()
        os._exit(0)


def read_traffic_from_profile():
    """DRAM bytes per launch of the GEMM kernel from the committed ncu summary, if one exists."""
    path = os.path.join(ROOT, "profiles", "w46_gemm_tc5_traffic.json")
    if os.path.isfile(path):
        with open(path) as f:
            return json.load(f).get("dram_bytes_per_launch_full_size")
    return None


def run_sweep(fm, synth, dev, peaks, only=None):
    """Latency / GB/s / TFLOP/s of other shapes (graph-timed like `value`); extra information."""
    import torch
    out = []
    shapes = [("cfg1", K_DIM, N_DIM, m) for m in (1, 2, 4, 8, 16, 32, 64, 128)]
    for name, (k, n) in synth.LLAMA2_7B.items():
        shapes += [(f"7b_{name}", k, n, m) for m in (1, 16, 128)]
    shapes += [("cfg4", 16384, 16384, m) for m in (1024, 4096)]      # tensor-bound: compare with the bf16 GEMM peak
    if only is not None:
        shapes = [("only",) + tuple(only)]
    cache = {}
    for tag, k, n, m in shapes:
        if (k, n) not in cache:
            cache.clear()
            wt = synth.make_layer(k, n, QUANT_COLS, GROUP, seed=1, keep_dequantized=False, quant_device=dev)
            ncopies = max(2, int(300e6 // (wt.B.numel() * 4)) + 1) if m < 1024 else 1   # large M re-streams B per 256 rows anyway
            cache[(k, n)] = [(wt.B.to(dev).clone(), wt.s.to(dev).clone()) for _ in range(ncopies)]
        copies = cache[(k, n)]
        a = synth.make_activations(m, k).to(dev)
        c = torch.zeros((m, n), dtype=torch.float16, device=dev)
        ws = torch.zeros(n // 128 * 16, dtype=torch.int32, device=dev)
        stream = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(stream):
            for i in range(5):
                fm.mul(a, *copies[i % len(copies)][:1], c, copies[i % len(copies)][1], ws, QUANT_COLS, group_size=GROUP, layout="b200")
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            reps = 200 if m <= 128 else 4
            with torch.cuda.graph(g, stream=stream):
                for i in range(reps):
                    B, s = copies[i % len(copies)]
                    fm.mul(a, B, c, s, ws, QUANT_COLS, group_size=GROUP, layout="b200")
            g.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(5):
                g.replay()
            e1.record(stream)
            torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (5 * reps)
        nbytes = synth.algorithmic_bytes(m, k, n, QUANT_COLS, GROUP)
        fl = synth.flops(m, k, n)
        out.append({"shape": tag, "M": m, "K": k, "N": n, "us": us, "GBs": nbytes / us / 1e3, "TFLOPs": fl / us / 1e6,
                    "hbm_frac": nbytes / us / 1e3 / peaks["hbm_gbs"],
                    "tensor_frac_sustained": fl / us / 1e6 / peaks["bf16_tflops_sustained"]})
    return out


def main():
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
    else:
        b200_arm(args)


if __name__ == "__main__":
    main()

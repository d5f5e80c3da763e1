#!/usr/bin/env python
"""Benchmark of the W(4&6)A16 GEMM path.

Workload (one "step" = one `mul` call): the square layer of the single-GPU sweep, K = N = 8192,
M = 16 rows of fp16 activations, 256 FP6 columns + INT4 group-128 elsewhere, seeded synthetic
values (fp6_marlin_b200/synth.py).  The metric is effective HBM bandwidth: algorithmic bytes of
one GEMM (A + packed weights + scales + C, the form of the reference's bench.py:46-50) divided by
its latency.

  value      the K steps captured in one CUDA graph (the launch-bound inner loop), inputs resident in
             HBM, each step on a different one of several weight copies so that the working set exceeds
             L2.  The graph is replayed until at least 0.4 s have been timed (CUDA events on the launching
             stream around every replay); `ms_per_step` is the median replay divided by K.
  e2e        the same K steps through the public Python API with HOST buffers: every step copies A
             from pinned host memory, calls mul, and copies C back to pinned host memory.
  roofline   achieved GB/s of one GPU's GEMM kernel in the timed region against the measured HBM peak
             (MEASURED_PEAKS.json); `traffic` is the DRAM byte count of one launch from an ncu capture.
  sweep      (1 GPU) the other points of the configurations: the square layer at M = 1, 16, 64, 128, the
             Llama-2-7B layers at M = 16 and the compute-bound layer K = N = 16384 at M = 1024, each
             with latency, GB/s, TFLOP/s, fractions of the measured peaks and a relative Frobenius error
             of a column subset against the CPU oracle (checker only).
  fused_epilogue
             (1 GPU) the Llama-2-7B gate / up projection at M = 16: `mul_fused` with the SiLU * up epilogue against
             the unfused GEMM followed by torch kernels.
  multi      (N > 1) GEMM alone / exchange alone / fused per step, a Llama-2-70B gate_up shard at M = 16
             and, on 8 GPUs, the compute-bound layer at M = 8192.
  cpu_baseline / --impl reference
             the reference's CPU path for the same layer - FP6 columns dequantised by the
             reference's own host code (oracle/_ref), INT4 columns by the rule of its test script
             ((q-8).half()*s), then torch.matmul in fp32 - timed on the host cores.

With N > 1 GPUs (torchrun) the layer's output columns are sharded over the ranks and every step
ends with the all-gather of the output columns (fused into the GEMM epilogue as peer stores, or NCCL):
total work is fixed ("strong" scaling).
"""
from __future__ import annotations

import argparse
import json
import math
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
WORKLOAD = "cfg1 square layer K=N=8192 M=16 qc=256 INT4-g128"
UNIT = "GB/s"
MIN_TIMED_MS = 400.0       # the K-step graph is replayed until this much has been timed
L2_BYTES = 126e6


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-sweep", action="store_true", help="skip the other M values and layer shapes (1 GPU)")
    ap.add_argument("--full-sweep", action="store_true", help="every M of every configuration that fits one GPU")
    ap.add_argument("--no-multi", action="store_true", help="N > 1: skip the extra shapes and the part timings")
    ap.add_argument("--multi-cfg4", action="store_true", help="N > 1: time the compute-bound layer at M = 8192 also on fewer than 8 GPUs")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: all-gather of the output columns fused into the GEMM epilogue as peer stores, or NCCL")
    ap.add_argument("--only-shape", default=None, metavar="K,N,M[,qc]",
                    help="time just this shape the way the sweep does and print its record (used for profiling other shapes)")
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
        self.marks = []          # (t_begin, t_end) of the timed regions, host clock
        self.proc = None
        cmd = ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50"]
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
                self.rows.append((time.perf_counter(), parts))

    def mark(self, t0, t1):
        self.marks.append((t0, t1))

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, sm_max, reasons, in_region = [], [], set(), []
        for t, r in self.rows:
            try:
                v = float(r[1])
                sm_max.append(float(r[2]))
            except ValueError:
                continue
            sm.append(v)
            timed = any(a <= t <= b + 0.06 for a, b in self.marks)
            if timed:
                in_region.append(v)
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        # samples taken while a timed region ran; if the sampler missed them all, those in the upper half
        load = in_region or ([x for x in sm if x >= 0.5 * max(sm)] if sm else [])
        return {"sm_mhz": statistics.median(load) if load else None,
                "sm_max_mhz": max(sm_max) if sm_max else None,
                "samples": len(sm), "samples_in_timed_regions": len(in_region), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------
# the reference's CPU path (checker code: bench.py executes oracle/ here and in the sweep's checker)
# ------------------------------------------------------------------------------------------------
def cpu_reference_step_fn(n_int4_cols: int):
    """Returns (step(), algorithmic_bytes, kind, description) for the reference's CPU path on a column
    slab of the benchmark layer: `n_int4_cols` INT4 columns plus all 256 FP6 columns."""
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
    """Times the reference's CPU path on all host cores; sizes the column slab so that the run stays
    within budget."""
    import torch
    # torchrun exports OMP_NUM_THREADS=1: use the host's cores whatever the launcher set
    torch.set_num_threads(max(1, os.cpu_count() or 1))
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
        "data": "synthetic", "config": {"workload": WORKLOAD, "arm": "CPU path of the reference on the host cores"},
        "cpu_baseline": {"value": res["value"], "unit": UNIT, "cores": res["cores"], "kind": res["kind"], "sample": res["sample"]},
        "e2e": {"value": res["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# one layer on N GPUs
# ------------------------------------------------------------------------------------------------
class LayerBench:
    """One W(4&6)A16 layer, N-sharded over the ranks when world > 1, with everything a timed step needs."""

    def __init__(self, env, k, n, m, qc, gs, exchange_kind="peer", seed=0, weight_on_gpu=False, min_copy_bytes=280e6):
        import torch
        fm, shard, synth = env["fm"], env["shard"], env["synth"]
        self.env, self.k, self.n, self.m, self.qc, self.gs = env, k, n, m, qc, gs
        dev, rank, world = env["dev"], env["rank"], env["world"]
        self.world = world
        self.n_local, self.qc_local = n // world, (qc // world if qc > 0 else qc)
        w = synth.make_weight_fp16(k, n, qc, seed=seed, device=dev if weight_on_gpu else None)
        self.w_full_fp16 = w if not weight_on_gpu else None
        self.plan = shard.ShardPlan(n, max(qc, 0), world)
        if world > 1:
            w = shard.shard_weight(w, self.plan, rank)
        self.w_local_fp16 = w
        weight = fm.make_w46_weight(w, self.qc_local, gs, keep_dequantized=False, quant_device=dev)
        self.weight = weight
        per_copy = weight.B.numel() * 4
        n_copies = max(2, int(min_copy_bytes // per_copy) + 1) if min_copy_bytes > 0 else 1
        self.copies = [(weight.B.to(dev).clone(), weight.s.to(dev).clone()) for _ in range(n_copies)]
        self.copy_bytes = n_copies * per_copy
        self.a_host = synth.make_activations(m, k).pin_memory()
        self.a_dev = self.a_host.to(dev)
        self.c_dev = torch.zeros((m, self.n_local), dtype=torch.float16, device=dev)
        self.gathered = torch.zeros((world, m, self.n_local), dtype=torch.float16, device=dev) if world > 1 else None
        self.c_host = torch.zeros((m, n), dtype=torch.float16).pin_memory()
        self.workspace = torch.zeros(max(self.n_local // 128 * 16, 64), dtype=torch.int32, device=dev)
        self.stream = env["stream"]
        self.exchange = None
        self.exchange_kind = exchange_kind if world > 1 else None
        if world > 1 and exchange_kind == "peer":
            from types import SimpleNamespace
            self.exchange = shard.PeerExchange(self.plan, rank, m, dev)
            self.shards = [SimpleNamespace(B=B, s=s, quant_cols=self.qc_local, group_size=gs) for B, s in self.copies]

    # ---- steps
    def gemm_only(self, i, a):
        B, s = self.copies[i % len(self.copies)]
        self.env["fm"].mul(a, B, self.c_dev, s, self.workspace, self.qc_local, group_size=self.gs, layout="b200")

    def step(self, i, a):
        import torch.distributed as dist
        if self.exchange is not None:
            # every rank stores its columns into every rank's (M, N) output; signal + bounded wait complete the step
            self.exchange.mul_scatter(a, self.shards[i % len(self.copies)], self.workspace, i % 2)
            self.exchange.finish()
            return
        self.gemm_only(i, a)
        if self.world > 1:
            dist.all_gather_into_tensor(self.gathered, self.c_dev)

    def exchange_only(self, i):
        import torch.distributed as dist
        if self.exchange is not None:
            self.exchange.finish()
        elif self.world > 1:
            dist.all_gather_into_tensor(self.gathered, self.c_dev)

    def launches_per_step(self):
        # the library's own launch plan for this shape and device
        import torch
        sms = torch.cuda.get_device_properties(self.env["dev"]).multi_processor_count
        per_gemm, _ = self.env["fm"].launch_plan(self.m, self.n_local, self.k, self.qc_local, sms)
        return per_gemm + (1 if self.exchange is not None else 0)

    # ---- timing
    def barrier(self):
        import torch
        import torch.distributed as dist
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def time_graph(self, fn, steps, min_ms=MIN_TIMED_MS, max_replays=400, sampler=None):
        """Captures `steps` calls of fn(i) in one CUDA graph and replays it until min_ms have been timed.
        Returns the per-replay times in ms (max over ranks for each replay)."""
        import torch
        import torch.distributed as dist
        stream = self.stream
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for i in range(steps):
                fn(i)
        g.replay()
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        g.replay()
        e1.record(stream)
        self.barrier()
        est = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=self.env["dev"])
        if self.world > 1:
            dist.all_reduce(est, op=dist.ReduceOp.MAX)
        replays = int(min(max_replays, max(3, math.ceil(min_ms / max(float(est.item()), 1e-3)))))
        events = [torch.cuda.Event(enable_timing=True) for _ in range(replays + 1)]
        self.barrier()
        t0 = time.perf_counter()
        events[0].record(stream)
        for j in range(replays):
            g.replay()
            events[j + 1].record(stream)
        self.barrier()
        t1 = time.perf_counter()
        if sampler is not None:
            sampler.mark(t0, t1)
        times = torch.tensor([events[j].elapsed_time(events[j + 1]) for j in range(replays)], dtype=torch.float64,
                             device=self.env["dev"])
        if self.world > 1:
            dist.all_reduce(times, op=dist.ReduceOp.MAX)
        del g
        return times.tolist()

    def time_e2e(self, steps, repeats=5):
        """`steps` steps through the public API with host buffers, host<->device copies inside; median of
        `repeats` such regions, ms per step (max over ranks)."""
        import torch
        import torch.distributed as dist
        stream = self.stream

        def one(i):
            self.a_dev.copy_(self.a_host, non_blocking=True)
            self.step(i, self.a_dev)
            if self.exchange is not None:
                self.c_host.copy_(self.exchange.outputs[i % 2], non_blocking=True)
            elif self.world > 1:
                self.c_host.view(self.world, self.m, self.n_local).copy_(self.gathered, non_blocking=True)    # rank-major blocks
            else:
                self.c_host.copy_(self.c_dev, non_blocking=True)

        for i in range(3):
            one(i)
        out = []
        for _ in range(repeats):
            self.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for i in range(steps):
                one(i)
            e1.record(stream)
            self.barrier()
            out.append(e0.elapsed_time(e1) / steps)
        t = torch.tensor(out, dtype=torch.float64, device=self.env["dev"])
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return statistics.median(t.tolist())

    def time_e2e_pipelined(self, steps, min_ms=200.0):
        """One GPU: the serving loop around the public `mul` with HOST buffers, software-pipelined over three
        streams and two device buffers: the host->device copy of step i + 1 and the device->host copy of step
        i - 1 overlap the GEMM of step i.  Every step still copies its A from pinned host memory and its C back.
        The `steps` steps are captured in one CUDA graph (copies are memcpy nodes of the graph) and replayed;
        if capture fails the same loop runs eagerly.  Returns (ms per step, mode)."""
        import torch
        fm = self.env["fm"]
        dev = self.env["dev"]
        s_mm = self.stream
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        a_devs = [self.a_dev, torch.empty_like(self.a_dev)]
        c_devs = [self.c_dev, torch.empty_like(self.c_dev)]
        c_hosts = [self.c_host, torch.empty_like(self.c_host).pin_memory()]

        def run(n_steps):
            fork = torch.cuda.Event()
            fork.record(s_mm)
            s_in.wait_event(fork)
            s_out.wait_event(fork)
            ev_in, ev_mm, ev_out = [None, None], [None, None], [None, None]
            for i in range(n_steps):
                b = i & 1
                with torch.cuda.stream(s_in):
                    if ev_mm[b] is not None:
                        s_in.wait_event(ev_mm[b])              # the GEMM of step i - 2 has read this buffer
                    a_devs[b].copy_(self.a_host, non_blocking=True)
                    ev_in[b] = torch.cuda.Event()
                    ev_in[b].record(s_in)
                with torch.cuda.stream(s_mm):
                    s_mm.wait_event(ev_in[b])
                    if ev_out[b] is not None:
                        s_mm.wait_event(ev_out[b])             # the result of step i - 2 has left this buffer
                    B, sc = self.copies[i % len(self.copies)]
                    fm.mul(a_devs[b], B, c_devs[b], sc, self.workspace, self.qc_local, group_size=self.gs, layout="b200")
                    ev_mm[b] = torch.cuda.Event()
                    ev_mm[b].record(s_mm)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_mm[b])
                    c_hosts[b].copy_(c_devs[b], non_blocking=True)
                    ev_out[b] = torch.cuda.Event()
                    ev_out[b].record(s_out)
            for e in ev_in + ev_out:                            # join
                if e is not None:
                    s_mm.wait_event(e)

        with torch.cuda.stream(s_mm):
            run(4)
        torch.cuda.synchronize()
        mode = "graph of the pipelined steps (memcpy nodes + GEMM), replayed"
        graph = None
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=s_mm):
                run(steps)
            graph.replay()
            torch.cuda.synchronize()
        except Exception as exc:          # noqa: BLE001 - capture of cross-stream copies is an optimisation only
            sys.stderr.write(f"e2e: graph capture of the pipelined loop failed ({exc}); running it eagerly\n")
            graph = None
            mode = "eager pipelined loop"
            torch.cuda.synchronize()
        times = []
        total = 0.0
        while total < min_ms and len(times) < 200:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(s_mm):
                e0.record(s_mm)
                if graph is not None:
                    graph.replay()
                else:
                    run(steps)
                e1.record(s_mm)
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
            total += times[-1]
        ok = bool(torch.equal(c_hosts[(steps - 1) & 1], c_devs[(steps - 1) & 1].cpu()))
        del graph
        return statistics.median(times) / steps, mode, ok

    def host_us_per_call(self, calls=2000):
        """Host time to enqueue one mul (Python + ctypes + tensor-map encoding + launch), device kept busy."""
        import torch
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(calls):
            self.gemm_only(i, self.a_dev)
        t1 = time.perf_counter()
        torch.cuda.synchronize()
        return (t1 - t0) / calls * 1e6

    def check_exchange(self, i):
        """Parity of the fused exchange: the same step through the NCCL all-gather + column assembly."""
        import torch
        import torch.distributed as dist
        shard, fm = self.env["shard"], self.env["fm"]
        # both GEMMs with one issuing thread per accumulator tile: bit-identical from run to run, so the two
        # paths can be compared for equality
        before = fm.set_ordered_sums(True)
        self.barrier()
        self.step(i, self.a_dev)
        self.gemm_only(i, self.a_dev)
        dist.all_gather_into_tensor(self.gathered, self.c_dev)
        expect = shard.assemble(self.gathered, self.plan)
        torch.cuda.synchronize()
        fm.set_ordered_sums(before)
        ok = torch.tensor([int(torch.equal(expect, self.exchange.outputs[i % 2]))], device=self.env["dev"])
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        return bool(ok.item())

    def close(self):
        import torch.distributed as dist
        if self.exchange is not None:
            self.barrier()
            self.exchange.close()
            dist.barrier()
            self.exchange = None


def oracle_subset_error(env, lb, n_cols=64):
    """Relative Frobenius error of a column subset of C (first INT4 columns, last FP6 columns) against the
    CPU oracle: oracle quantisation of those columns of the fp16 weights, fp32-accumulated product.
    Checker only; the product computes nothing here."""
    import numpy as np
    import torch
    from oracle import formats as F
    w = lb.w_local_fp16
    n_loc = lb.n_local
    qc = max(lb.qc_local, 0)
    rows = min(lb.m, 16)
    lb.gemm_only(0, lb.a_dev)
    torch.cuda.synchronize()
    c = lb.c_dev[:rows].float().cpu().numpy()
    a = lb.a_host[:rows].numpy()
    parts, cols = [], []
    n4 = min(n_cols, n_loc - qc)
    if n4 > 0:
        w4 = w[:, :n4].cpu().numpy()
        parts.append((F.int4_quantize_group(w4, 128) if lb.gs > 0 else F.int4_quantize_per_channel(w4))[2])
        cols += list(range(n4))
    n6 = min(n_cols, qc)
    if n6 > 0:
        w6 = w[:, n_loc - n6:].cpu().numpy()
        parts.append(F.fp6_codes_and_dequant(w6)[2])
        cols += list(range(n_loc - n6, n_loc))
    ref = F.gemm_reference(a, np.concatenate(parts, axis=1))
    return F.rel_frobenius(c[:, cols], ref)


def sweep_record(env, tag, k, n, m, qc, peaks, check=True):
    """Latency / GB/s / TFLOP/s of one shape (graph-timed like `value`) and its oracle check."""
    synth = env["synth"]
    sys.stderr.write(f"sweep: {tag} K={k} N={n} M={m} qc={qc}\n")
    sys.stderr.flush()
    lb = LayerBench(env, k, n, m, qc, GROUP, seed=1, weight_on_gpu=True,
                    min_copy_bytes=(300e6 if m < 1024 else 0))     # large M re-streams B per 256 rows anyway
    import torch
    with torch.cuda.stream(env["stream"]):
        for i in range(3):
            lb.gemm_only(i, lb.a_dev)
        torch.cuda.synchronize()
        err = oracle_subset_error(env, lb) if check else None
        reps = 100 if m <= 128 else 4
        times = lb.time_graph(lambda i: lb.gemm_only(i, lb.a_dev), reps, min_ms=60.0, max_replays=50)
    us = statistics.median(times) * 1e3 / reps
    nbytes = synth.algorithmic_bytes(m, k, n, qc, GROUP)
    fl = synth.flops(m, k, n)
    rec = {"shape": tag, "M": m, "K": k, "N": n, "qc": qc, "us": round(us, 2), "GBs": round(nbytes / us / 1e3, 1),
           "TFLOPs": round(fl / us / 1e6, 1), "hbm_frac": round(nbytes / us / 1e3 / peaks["hbm_gbs"], 3),
           "tensor_frac": round(fl / us / 1e6 / peaks["bf16_tflops"], 3),
           "tensor_frac_sustained": round(fl / us / 1e6 / peaks["bf16_tflops_sustained"], 3)}
    if err is not None:
        rec["rel_frobenius_vs_oracle"] = float(f"{err:.3e}")
    del lb
    torch.cuda.empty_cache()
    return rec


def fused_record(env, peaks, m=16):
    """The Llama-2-7B gate / up projection at M rows: one GEMM whose epilogue computes silu(gate) * up on the
    fp32 sums (`mul_fused`) against the unfused sequence - the same GEMM writing (M, 2I), then silu * up as
    torch kernels on the interleaved pairs."""
    import torch
    import torch.nn.functional as Fn
    fm, synth, dev = env["fm"], env["synth"], env["dev"]
    k, n = synth.LLAMA2_7B["gate_up"]
    inter = n // 2
    sys.stderr.write(f"sweep: fused gate_up K={k} I={inter} M={m}\n")
    gen = torch.Generator(device=dev).manual_seed(11)
    w_gate = (torch.randn((k, inter), generator=gen, device=dev) * 0.02).half()
    w_up = (torch.randn((k, inter), generator=gen, device=dev) * 0.02).half()
    w_gate[:, torch.randperm(inter, generator=gen, device=dev)[: QUANT_COLS // 2]] *= 8.0
    weight, _ = fm.make_gate_up_weight(w_gate, w_up, QUANT_COLS, GROUP, quant_device=dev)
    per_copy = weight.B.numel() * 4
    copies = [(weight.B.to(dev).clone(), weight.s.to(dev).clone()) for _ in range(int(300e6 // per_copy) + 1)]
    a = synth.make_activations(m, k).to(dev)
    c_fused = torch.zeros((m, inter), dtype=torch.float16, device=dev)
    c_full = torch.zeros((m, n), dtype=torch.float16, device=dev)
    c_act = torch.zeros((m, inter), dtype=torch.float16, device=dev)
    workspace = torch.zeros(max(n // 128 * 16, 64), dtype=torch.int32, device=dev)

    def fused(i):
        B, sc = copies[i % len(copies)]
        fm.mul_fused(a, B, c_fused, sc, workspace, QUANT_COLS, epilogue="silu_mul", group_size=GROUP)

    def unfused(i):
        B, sc = copies[i % len(copies)]
        fm.mul(a, B, c_full, sc, workspace, QUANT_COLS, group_size=GROUP, layout="b200")
        pairs = c_full.view(m, inter, 2)
        torch.mul(Fn.silu(pairs[:, :, 0]), pairs[:, :, 1], out=c_act)

    lb = LayerBench.__new__(LayerBench)          # only its graph timer is used
    lb.env, lb.world, lb.stream = env, 1, env["stream"]
    reps = 100
    with torch.cuda.stream(env["stream"]):
        for i in range(3):
            fused(i)
            unfused(i)
        torch.cuda.synchronize()
        same = float((c_fused.float() - c_act.float()).norm() / c_act.float().norm())
        t_fused = statistics.median(lb.time_graph(fused, reps, min_ms=60.0, max_replays=50)) * 1e3 / reps
        t_unfused = statistics.median(lb.time_graph(unfused, reps, min_ms=60.0, max_replays=50)) * 1e3 / reps
    del copies
    torch.cuda.empty_cache()
    return {"shape": "7b_gate_up", "M": m, "K": k, "N": n, "qc": QUANT_COLS, "fused_silu_mul_us": round(t_fused, 2),
            "unfused_gemm_then_torch_silu_mul_us": round(t_unfused, 2),
            "rel_difference_fused_vs_unfused": float(f"{same:.3e}")}


def run_sweep(env, peaks, full=False, only=None):
    synth = env["synth"]
    if only is not None:
        k, n, m = only[:3]
        qc = only[3] if len(only) > 3 else QUANT_COLS
        return [sweep_record(env, "only", k, n, m, qc, peaks)]
    shapes = [("cfg1", K_DIM, N_DIM, m, QUANT_COLS) for m in ((1, 2, 4, 8, 16, 32, 64, 128) if full else (1, 64, 128))]
    for name, (k, n) in synth.LLAMA2_7B.items():
        shapes += [(f"7b_{name}", k, n, m, QUANT_COLS) for m in ((1, 16, 128) if full else (16,))]
    if full:
        shapes += [("cfg4", 16384, 16384, m, qc) for m in (1024, 2048, 4096, 8192) for qc in ((0, 128, 256, 512) if m == 1024 else (256,))]
    else:
        shapes += [("cfg4", 16384, 16384, 1024, 256)]
    return [sweep_record(env, tag, k, n, m, qc, peaks) for tag, k, n, m, qc in shapes]


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
    peaks = measured_peaks()
    env = {"fm": fm, "shard": shard, "synth": synth, "dev": dev, "rank": rank, "world": world,
           "stream": torch.cuda.Stream(device=dev)}
    # consecutive GEMMs of a decode step: each may set itself up and prefetch its (static) weights while
    # the previous kernel of the stream drains; activations, outputs and scratch wait for that kernel
    fm.set_launch_overlap(not args.no_overlap)
    if args.only_shape:
        only = tuple(int(x) for x in args.only_shape.split(","))
        env["world"] = 1
        print(json.dumps(run_sweep(env, peaks, only=only)[0]))
        return
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    assert world == args.gpus or world == 1, "launch with torchrun --nproc-per-node == --gpus"

    steps, warmup = args.steps, max(args.warmup, 3)
    sampler = ClockSampler(str(torch.cuda.get_device_properties(dev).uuid)) if rank == 0 else None
    lb = LayerBench(env, K_DIM, N_DIM, M_ROWS, QUANT_COLS, GROUP, exchange_kind=args.exchange, seed=0)
    multi = None
    with torch.cuda.stream(env["stream"]):
        for i in range(warmup):
            lb.step(i, lb.a_dev)
        torch.cuda.synchronize()
        exchange_ok = lb.check_exchange(warmup - 1) if lb.exchange is not None else None
        times = lb.time_graph(lambda i: lb.step(i, lb.a_dev), steps, sampler=sampler)
        ms_e2e = lb.time_e2e(steps)
        e2e_pipe = lb.time_e2e_pipelined(steps) if world == 1 else None
        host_us = lb.host_us_per_call() if world == 1 else None
        if world > 1 and not args.no_multi:
            multi = multi_gpu_extras(env, lb, args, peaks)
    clocks = sampler.stop() if sampler else None
    status = fm.device_status(dev)

    nbytes = synth.algorithmic_bytes(M_ROWS, K_DIM, N_DIM, QUANT_COLS, GROUP)                      # whole layer
    nbytes_local = synth.algorithmic_bytes(M_ROWS, K_DIM, lb.n_local, max(lb.qc_local, 0), GROUP)   # one rank's kernel
    ms_step = statistics.median(times) / steps
    value = nbytes / (ms_step * 1e-3) / 1e9
    achieved = nbytes_local / (ms_step * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp16 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": WORKLOAD, "M": M_ROWS, "K": K_DIM, "N": N_DIM, "quant_cols": QUANT_COLS, "group_size": GROUP,
                   "l2": f"{len(lb.copies)} rotating weight copies ({lb.copy_bytes / 1e6:.0f} MB) exceed L2",
                   "parallelism": "single GPU" if world == 1 else (
                       f"N-sharded over {world} GPUs, output columns exchanged by peer stores in the GEMM epilogue + signal/wait kernels"
                       if lb.exchange is not None else f"N-sharded over {world} GPUs + NCCL all-gather of output columns"),
                   "graph": True, "launch_overlap": not args.no_overlap,
                   "timing": f"graph of {steps} steps replayed {len(times)} times; median replay / steps",
                   "ms_per_step_min": min(times) / steps, "ms_per_step_max": max(times) / steps},
        "e2e": {"value": nbytes / (ms_e2e * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": lb.a_host.numel() * 2, "d2h_bytes_per_step": M_ROWS * N_DIM * 2},
        "gpu_launches": steps * len(times) * lb.launches_per_step(),
        "gpu_launches_per_step": lb.launches_per_step(),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "peak_source": f"of {peaks['source']}",
                     "algorithmic_bytes": nbytes_local, "per": "GPU" if world > 1 else "launch",
                     "traffic": read_traffic_from_profile() if world == 1 else None},
        "clocks": clocks,
        "device_status": status,
    }
    if e2e_pipe is not None:
        # the headline end-to-end number is the pipelined serving loop; the strictly serial loop stays beside it
        line["e2e"].update({"serial_ms_per_step": ms_e2e, "serial_value": line["e2e"]["value"],
                            "ms_per_step": e2e_pipe[0], "value": nbytes / (e2e_pipe[0] * 1e-3) / 1e9,
                            "mode": "host->device copy of step i+1 and device->host copy of step i-1 overlap the GEMM of step i "
                                    "(three streams, two device buffers); " + e2e_pipe[1],
                            "result_on_host_matches_device": e2e_pipe[2]})
    if host_us is not None:
        line["e2e"]["host_us_per_mul_call"] = host_us
    if exchange_ok is not None:
        line["config"]["exchange_matches_nccl_all_gather"] = exchange_ok
    if multi is not None:
        line["multi"] = multi
    lb.close()
    del lb
    torch.cuda.empty_cache()
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cb = time_cpu_reference(steps=5, warmup=1, budget_s=25.0)
        line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
    if world == 1 and not args.no_sweep:
        with torch.cuda.stream(env["stream"]):
            line["sweep"] = run_sweep(env, peaks, full=args.full_sweep)
        line["fused_epilogue"] = fused_record(env, peaks)
        line["device_status"] = line["device_status"] or fm.device_status(dev)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        # CUDA graphs that captured NCCL work must go before the communicator does; a watchdog ends the
        # process if the tear-down of the process group stalls (the result line is already printed)
        torch.cuda.synchronize()
        sys.stdout.flush()
        threading.Timer(20.0, lambda: os._exit(0)).start()
        dist.barrier()
        dist.destroy_process_group()
        os._exit(0)


def multi_gpu_extras(env, lb, args, peaks):
    """N > 1: where a step's time goes for the headline layer, plus the shapes where sharding divides real
    work: a Llama-2-70B gate_up layer at M = 16 and (8 GPUs) the compute-bound layer at M = 8192."""
    import torch
    synth = env["synth"]
    world = env["world"]
    out = {}
    reps = 200
    t_gemm = statistics.median(lb.time_graph(lambda i: lb.gemm_only(i, lb.a_dev), reps, min_ms=100.0)) * 1e3 / reps
    t_xchg = statistics.median(lb.time_graph(lambda i: lb.exchange_only(i), reps, min_ms=50.0)) * 1e3 / reps
    t_fused = statistics.median(lb.time_graph(lambda i: lb.step(i, lb.a_dev), reps, min_ms=100.0)) * 1e3 / reps
    out["headline_parts_us"] = {"gemm_us": t_gemm, "exchange_us": t_xchg, "fused_us": t_fused,
                                "exchange": lb.exchange_kind}

    def shape_record(tag, k, n, m, qc, reps, min_ms):
        b = LayerBench(env, k, n, m, qc, GROUP, exchange_kind=args.exchange, seed=2, weight_on_gpu=True,
                       min_copy_bytes=(300e6 if m <= 128 else 0))
        for i in range(3):
            b.step(i, b.a_dev)
        torch.cuda.synchronize()
        ok = b.check_exchange(2) if b.exchange is not None else None
        tg = statistics.median(b.time_graph(lambda i: b.gemm_only(i, b.a_dev), reps, min_ms=min_ms)) * 1e3 / reps
        tf = statistics.median(b.time_graph(lambda i: b.step(i, b.a_dev), reps, min_ms=min_ms)) * 1e3 / reps
        nbytes_local = synth.algorithmic_bytes(m, k, b.n_local, max(b.qc_local, 0), GROUP)
        fl = synth.flops(m, k, n)
        rec = {"shape": tag, "M": m, "K": k, "N": n, "qc": qc, "gemm_us": tg, "fused_us": tf,
               "aggregate_GBs": world * nbytes_local / tf / 1e3, "aggregate_TFLOPs": fl / tf / 1e6,
               "per_gpu_hbm_frac": nbytes_local / tf / 1e3 / peaks["hbm_gbs"],
               "per_gpu_tensor_frac": fl / world / tf / 1e6 / peaks["bf16_tflops"],
               "exchange_matches_nccl_all_gather": ok}
        b.close()
        del b
        torch.cuda.empty_cache()
        return rec

    k, n = synth.LLAMA2_70B["gate_up"]
    out["cfg3_70b_gate_up_m16"] = shape_record("70b_gate_up", k, n, 16, QUANT_COLS, 100, 60.0)
    if world == 8 or args.multi_cfg4:
        out["cfg4_m8192"] = shape_record("cfg4", 16384, 16384, 8192, QUANT_COLS, 2, 60.0)
    return out


def read_traffic_from_profile():
    """DRAM bytes per launch of the GEMM kernel from the committed ncu summary, if one exists."""
    path = os.path.join(ROOT, "profiles", "w46_gemm_tc5_traffic.json")
    if os.path.isfile(path):
        with open(path) as f:
            return json.load(f).get("dram_bytes_per_launch_full_size")
    return None


def main():
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
    else:
        b200_arm(args)


if __name__ == "__main__":
    main()

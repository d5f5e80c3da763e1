"""In-kernel timeline of the GEMM for up to 128 rows (developer tool; needs a B200).

The library built with ``python fp6_marlin_b200/build.py --trace`` records, in two CTAs of every launch,
{tag, argument, SM clock} events of every warp (csrc/trace.cuh), and the start and end of every CTA of the
last 64 launches in nanoseconds.  This module runs a few launches and prints both:

    FP6M_LIB=fp6_marlin_b200/libfp6m_trace.so python -m fp6_marlin_b200.timeline 8192,8192,16

``timeline``  per segment n of a traced CTA, in SM cycles since the CTA started: when its dequantiser team
              began it, found its ring entry free, had expanded it, had loaded the next segment's words, saw
              its tensor-memory stores drained and published it; when its MMA issuers started and finished;
              when an epilogue warp had its sums and had added them.
``launches``  for a CUDA graph of back-to-back launches with and without programmatic dependent launch:
              first / last CTA start and end of each launch, the CTA lifetime and the period between launches.
"""
from __future__ import annotations

import ctypes
import sys

import numpy as np
import torch

import fp6_marlin_b200 as fm
from fp6_marlin_b200 import _lib, synth

CTAS_TRACED, WARPS, ENTRIES = 2, 32, 1024


def _trace_fn(name):
    try:
        fn = getattr(_lib.lib, name)
    except AttributeError:
        raise SystemExit("this library has no timeline: build it with `python fp6_marlin_b200/build.py --trace` "
                         "and set FP6M_LIB=fp6_marlin_b200/libfp6m_trace.so")
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_size_t]
    return fn


def _problem(k, n, m, dev, copies=9):
    wt = synth.make_layer(k, n, 256, 128, seed=1, keep_dequantized=False, quant_device=dev)
    cs = [(wt.B.clone(), wt.s.clone()) for _ in range(copies)]
    a = synth.make_activations(m, k).to(dev)
    c = torch.zeros((m, n), dtype=torch.float16, device=dev)
    ws = torch.zeros(max(n // 128 * 16, 64), dtype=torch.int32, device=dev)
    return cs, a, c, ws


def timeline(k, n, m):
    dev = torch.device("cuda:0")
    read = _trace_fn("fp6m_trace_read")
    fm.set_launch_overlap(False)
    cs, a, c, ws = _problem(k, n, m, dev, copies=6)
    for i in range(6):
        fm.mul(a, cs[i][0], c, cs[i][1], ws, 256, group_size=128, layout="b200")
    torch.cuda.synchronize()
    buf = np.zeros((CTAS_TRACED, WARPS, ENTRIES), dtype=np.uint64)
    rc = read(buf.ctypes.data, buf.nbytes)
    print("trace_read rc", rc, "device status", fm.device_status(dev))
    teams = 3 if m <= 32 else 2          # dequantiser teams of the kernel instance for m rows
    deq = (2 + 2 * teams + 3) & ~3
    epi = deq + 4 * teams
    for ci in range(CTAS_TRACED):
        ev = {}
        for w in range(WARPS):
            cnt = int(buf[ci, w, 0])
            ev[w] = [(int(x >> 56), int((x >> 32) & 0xFFFFFF), int(x & 0xFFFFFFFF)) for x in buf[ci, w, 1:1 + cnt]]
        print(f"==== traced CTA #{ci} (cycles since the CTA started)")
        print("set-up: barriers initialised / after the CTA-wide barrier and the grid dependency:",
              [(t, tt) for (t, _, tt) in ev[1] if t in (2, 4)])
        print("a dequantiser warp during set-up: CTA range known (30) / its stage's barriers initialised (31) / copy source computed (32) / copy issued (1):",
              [(t, tt) for (t, _, tt) in ev[deq] if t in (30, 31, 32, 1)][:4])
        print("first round of weight copies issued at:", sorted(tt for w in range(deq, min(WARPS, deq + 16)) for (t, _, tt) in ev[w] if t == 1))
        print("weights producer, later copies:", [tt for (t, _, tt) in ev[0] if t == 1][:12], "...")
        iss = {}
        for w in range(2, 2 + 2 * teams):
            cur = {}
            for (t, a_, tt) in ev[w]:
                if t == 6:
                    cur[a_] = [tt, None]
                if t == 7 and a_ in cur:
                    cur[a_][1] = tt
            for kk, vv in cur.items():
                iss.setdefault(kk, []).append(tuple(vv))
        seg = {}
        for w in range(deq, epi, 4):
            last = None
            for (t, a_, tt) in ev[w]:
                if t == 10:
                    seg[a_] = {10: tt}
                    last = a_
                elif t in (12, 13, 17, 18, 19) and last is not None:
                    seg[last][t] = tt
        got = {}
        for (t, a_, tt) in ev[epi] + ev[epi + 4]:
            if t in (15, 16):
                got.setdefault(a_, {})[t] = tt
        print("  n |   top  free  expanded  next-loaded  drained  published | issuers (start, end) | epilogue has sums, added")
        for nn in sorted(seg):
            s, r = seg[nn], got.get(nn, {})
            print(f"{nn:3d} | {s.get(10)!s:>6} {s.get(12)!s:>6} {s.get(17)!s:>6} {s.get(18)!s:>6} {s.get(19)!s:>6} {s.get(13)!s:>6} | "
                  f"{iss.get(nn, [])!s:>44} | {r.get(15)!s:>7} {r.get(16)!s:>7}")
        print("end of a slice (20) / its sums written or stored as a partial (22) / past the strip reduction (23) / CTA end (24):",
              [(t, tt) for (t, _, tt) in ev[epi] if 20 <= t <= 24])
        for w in list(range(deq, deq + 8, 4)) + list(range(epi, min(WARPS, epi + 16), 4)):
            red = [(t, tt) for (t, _, tt) in ev[w] if t in (25, 26, 27)]
            if red:
                print(f"  strip reduction, warp {w}: entered (25) / a round's tagged words all present (26) / C written (27):", red)


def launches(k, n, m):
    dev = torch.device("cuda:0")
    read = _trace_fn("fp6m_launch_times_read")
    cs, a, c, ws = _problem(k, n, m, dev)
    for overlap in (False, True):
        fm.set_launch_overlap(overlap)
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            for i in range(5):
                fm.mul(a, cs[i % 9][0], c, cs[i % 9][1], ws, 256, group_size=128, layout="b200")
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for i in range(40):
                    fm.mul(a, cs[i % 9][0], c, cs[i % 9][1], ws, 256, group_size=128, layout="b200")
            g.replay()
            torch.cuda.synchronize()
            g.replay()
            torch.cuda.synchronize()
        buf = np.zeros((64, 160, 2), dtype=np.uint64)
        read(buf.ctypes.data, buf.nbytes)
        used = buf[:, :, 1].max(axis=0) > 0
        starts, ends = buf[:, used, 0].astype(np.int64), buf[:, used, 1].astype(np.int64)
        order = np.argsort(starts.min(axis=1))[-30:]
        t0 = starts[order[0]].min()
        print(f"programmatic dependent launch {'on' if overlap else 'off'} ({int(used.sum())} CTAs): microseconds")
        prev = None
        for e in order[:10]:
            s_, e_ = starts[e] - t0, ends[e] - t0
            line = (f"  launch: CTA starts {s_.min() / 1e3:7.2f}..{s_.max() / 1e3:7.2f}  CTA ends {e_.min() / 1e3:7.2f}..{e_.max() / 1e3:7.2f}"
                    f"  median CTA lifetime {np.median(e_ - s_) / 1e3:5.2f}")
            if prev is not None:
                line += f"  first start - previous last end {(s_.min() - prev) / 1e3:6.2f}"
            print(line)
            prev = e_.max()
        print(f"  mean period between launch ends: {np.diff(np.sort(ends[order].max(axis=1))).mean() / 1e3:.2f}")


if __name__ == "__main__":
    shape = tuple(int(x) for x in (sys.argv[1] if len(sys.argv) > 1 else "8192,8192,16").split(","))
    mode = sys.argv[2] if len(sys.argv) > 2 else "both"
    if mode in ("timeline", "both"):
        timeline(*shape)
    if mode in ("launches", "both"):
        launches(*shape)

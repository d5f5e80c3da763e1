"""A bounded wait that runs out: the hand-shake kernel of the fused all-gather waits for flags that nobody
sets.  The wait must give up after its limit, record FP6M_ERR_TIMEOUT in the device status word and leave
the context usable; the next GEMM must be correct.  Nothing here faults or hangs: the limit is shortened to
a fraction of a millisecond through fp6m_set_peer_wait_polls and the kernel simply returns.
The reference's counterpart, barrier_acquire, spins without limit (fp6_marlin_cuda_kernel.cu:79-86)."""
import time

import numpy as np
import pytest
import torch

import fp6_marlin_b200 as fm
from fp6_marlin_b200 import _lib, api, synth

pytestmark = pytest.mark.gpu


def test_wait_that_runs_out_sets_the_status_word_and_returns():
    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    lib = _lib.lib
    # a GEMM before, for comparison afterwards
    m, k, n, qc, gs = 16, 1024, 1024, 256, 128
    w = synth.make_layer(k, n, qc, gs, seed=8, keep_dequantized=False).to(dev)
    a = synth.make_activations(m, k, 8).to(dev)
    workspace = torch.zeros(n // 128 * 16, dtype=torch.int32, device=dev)
    before = torch.zeros((m, n), dtype=torch.float16, device=dev)
    ordered = fm.set_ordered_sums(True)          # fixed order of additions: the two GEMMs below can be compared bit for bit
    fm.mul(a, w.B, before, w.s, workspace, qc, group_size=gs, layout="b200")
    torch.cuda.synchronize()
    assert fm.device_status(dev) == 0
    _, _, status = api._device_buffers(dev)

    flags = torch.zeros(8, dtype=torch.int32, device=dev)          # two "ranks": nobody ever signals
    step = torch.full((1,), 5, dtype=torch.int32, device=dev)      # this rank is at step 5
    previous = lib.fp6m_set_peer_wait_polls(2000)                  # about 0.2 ms instead of half a second
    try:
        stream = torch.cuda.current_stream(dev).cuda_stream
        t0 = time.perf_counter()
        rc = lib.fp6m_peer_wait(flags.data_ptr(), 2, step.data_ptr(), status.data_ptr(), dev.index or 0, stream)
        assert rc == _lib.OK
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t0
    finally:
        lib.fp6m_set_peer_wait_polls(previous)
    assert elapsed < 0.5, elapsed                                  # it gave up by itself, quickly
    assert fm.device_status(dev) == _lib.ERR_TIMEOUT               # reading clears the word
    assert fm.device_status(dev) == 0

    # a wait whose flags are there returns without a status
    flags.fill_(5)
    rc = lib.fp6m_peer_wait(flags.data_ptr(), 2, step.data_ptr(), status.data_ptr(), dev.index or 0,
                            torch.cuda.current_stream(dev).cuda_stream)
    assert rc == _lib.OK
    torch.cuda.synchronize()
    assert fm.device_status(dev) == 0

    # the context is intact: the same GEMM gives the same bits
    after = torch.zeros((m, n), dtype=torch.float16, device=dev)
    fm.mul(a, w.B, after, w.s, workspace, qc, group_size=gs, layout="b200")
    torch.cuda.synchronize()
    fm.set_ordered_sums(ordered)
    assert torch.equal(before, after)
    assert fm.device_status(dev) == 0


@pytest.mark.parametrize("m", [16, 96, 300])
def test_long_predecessor_does_not_run_the_bounded_waits_out(m):
    """Launch overlap on, and the kernel before the GEMM runs for 2.5 s - longer than the ~1 s bound of the
    GEMM's own waits - after letting its dependents launch at once.  The GEMM's CTAs are resident all that
    time; their bounded waits must only start once the predecessor has finished: status 0, same result."""
    dev = torch.device("cuda:0")
    lib = _lib.lib
    k, n, qc, gs = 2048, 2048, 256, 128
    w = synth.make_layer(k, n, qc, gs, seed=9, keep_dequantized=False).to(dev)
    a = synth.make_activations(m, k, 9).to(dev)
    workspace = torch.zeros(n // 128 * 16, dtype=torch.int32, device=dev)
    ordered = fm.set_ordered_sums(True)
    overlap = fm.set_launch_overlap(False)
    try:
        expect = torch.zeros((m, n), dtype=torch.float16, device=dev)
        fm.mul(a, w.B, expect, w.s, workspace, qc, group_size=gs, layout="b200")
        torch.cuda.synchronize()
        fm.set_launch_overlap(True)
        c = torch.zeros((m, n), dtype=torch.float16, device=dev)
        stream = torch.cuda.current_stream(dev).cuda_stream
        t0 = time.perf_counter()
        assert lib.fp6m_debug_busy_kernel(2500, dev.index or 0, stream) == _lib.OK
        fm.mul(a, w.B, c, w.s, workspace, qc, group_size=gs, layout="b200")
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t0
    finally:
        fm.set_launch_overlap(overlap)
        fm.set_ordered_sums(ordered)
    assert 2.4 < elapsed < 4.0, elapsed
    assert fm.device_status(dev) == 0
    assert torch.equal(c, expect)

"""The allocation-free entry point, fp6m_mul_static_scratch, called through the C ABI.

Some users of this library cannot hand it a scratch buffer because they cannot allocate one: a
plug-in inside a serving runtime that owns the whole device arena, or a loop that runs after the
allocator has been frozen.  For them the library carries its split-K scratch as a static array.
This test checks that the entry point gives the same answer as fp6m_mul (which takes a caller's
scratch buffer) - twice in a row, because every call reuses the same array and must not depend on
what the previous call left in it.  The file name makes pytest collect it last.
"""
import ctypes

import pytest
import torch

import fp6_marlin_b200 as fm
from fp6_marlin_b200 import _lib, synth

pytestmark = pytest.mark.gpu


def _call_static(a, w, c, workspace, qc, gs, sms=-1):
    stream = torch.cuda.current_stream(a.device).cuda_stream
    return _lib.lib.fp6m_mul_static_scratch(
        a.data_ptr(), w.B.data_ptr(), c.data_ptr(), w.s.data_ptr(), a.shape[0], c.shape[1], a.shape[1],
        workspace.data_ptr(), workspace.numel() * workspace.element_size(), a.device.index or 0, stream,
        -1, -1, sms, 16, qc, gs, _lib.LAYOUT_B200, None)


def test_static_scratch_entry_point_matches_mul_twice():
    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    m, k, n, qc, gs = 16, 2048, 4096, 256, 128          # several CTAs share every strip: the scratch is used
    w = synth.make_layer(k, n, qc, gs, seed=5, keep_dequantized=False).to(dev)
    a = synth.make_activations(m, k, 5).to(dev)
    workspace = torch.zeros(n // 128 * 16, dtype=torch.int32, device=dev)
    expected = torch.zeros((m, n), dtype=torch.float16, device=dev)
    # with ordered sums the kernel adds in one fixed order, so that the two entry points can be compared bit for bit
    previous = fm.set_ordered_sums(True)
    try:
        fm.mul(a, w.B, expected, w.s, workspace, qc, group_size=gs, layout="b200")
        torch.cuda.synchronize()
        assert float(expected.float().abs().sum()) > 0
        for attempt in range(2):
            got = torch.full((m, n), float("nan"), dtype=torch.float16, device=dev)
            rc = _call_static(a, w, got, workspace, qc, gs)
            torch.cuda.synchronize()
            assert rc == _lib.OK, (attempt, rc, _lib.last_cuda_error())
            # same kernel, same schedule, fixed summation order: the two entry points agree bit for bit,
            # which is well inside the 1e-3 relative tolerance the other GPU tests use
            err = (torch.linalg.norm(got.float() - expected.float()) / torch.linalg.norm(expected.float())).item()
            assert err <= 1e-3, (attempt, err)
            assert torch.equal(got, expected), attempt
    finally:
        fm.set_ordered_sums(previous)
    # and in the default mode, where the halves of a block may be added in either order, within the tolerance
    got = torch.full((m, n), float("nan"), dtype=torch.float16, device=dev)
    assert _call_static(a, w, got, workspace, qc, gs) == _lib.OK
    torch.cuda.synchronize()
    err = (torch.linalg.norm(got.float() - expected.float()) / torch.linalg.norm(expected.float())).item()
    assert err <= 1e-3, err
    assert int(workspace.abs().sum()) == 0
    assert fm.device_status(dev) == 0


def test_static_scratch_rejects_what_does_not_fit():
    dev = torch.device("cuda:0")
    m, k, n = 64, 4096, 8192                            # 64 rows on a full grid need more than 16 MiB
    w = synth.make_layer(k, n, 256, 128, seed=6, keep_dequantized=False).to(dev)
    a = synth.make_activations(m, k, 6).to(dev)
    c = torch.zeros((m, n), dtype=torch.float16, device=dev)
    workspace = torch.zeros(n // 128 * 16, dtype=torch.int32, device=dev)
    assert _call_static(a, w, c, workspace, 256, 128) == _lib.ERR_SCRATCH
    assert _call_static(a, w, c, workspace, 256, 128, sms=32) == _lib.OK    # a smaller grid fits
    torch.cuda.synchronize()

"""GPU parity tests of the GEMM, through the C ABI (libfp6m.so) behind the reference-shaped Python
API.  The checker is the oracle: W_deq from oracle/formats.py and C = A.float() @ W_deq.float()
accumulated in fp32 on the CPU.  Tolerance: relative Frobenius error <= 1e-3 (the bar the
benchmark configuration states; the reference's own tests use mean|dC|/mean|C| < 1e-3, test.py:181).
Shapes follow the reference's tests (test.py:183-237) plus the sharded and ragged cases of the
multi-GPU configurations."""
import os

import numpy as np
import pytest
import torch

import fp6_marlin
import fp6_marlin_b200 as fm
from fp6_marlin_b200 import synth
from oracle import formats as F

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _dev():
    assert torch.cuda.is_available(), "these tests need a CUDA GPU"
    return torch.device("cuda:0")


def _oracle_weight(w: torch.Tensor, qc: int, gs: int):
    """W_deq by the oracle's rules, from the fp16 weights."""
    k, n = w.shape
    nq = max(qc, 0)
    parts = []
    if n - nq:
        fn = (lambda x: F.int4_quantize_group(x, 128)) if gs > 0 else F.int4_quantize_per_channel
        parts.append(fn(w[:, : n - nq].numpy())[2])
    if nq:
        parts.append(F.fp6_codes_and_dequant(w[:, n - nq:].numpy())[2])
    return np.concatenate(parts, axis=1)


def _run(m, k, n, qc, gs, thread_k=-1, thread_n=-1, seed=0, sms=-1):
    dev = _dev()
    w = synth.make_weight_fp16(k, n, qc, seed)
    ww = fm.make_w46_weight(w, qc, gs, keep_dequantized=False).to(dev)
    a = synth.make_activations(m, k, seed)
    c = torch.zeros((m, n), dtype=torch.float16, device=dev)
    workspace = torch.zeros(max(n // 128 * 16, 16), device=dev)       # float32 zeros, as test.py:168
    fm.mul(a.to(dev), ww.B, c, ww.s, workspace, qc, thread_k, thread_n, sms, 16, group_size=gs, layout="b200")
    torch.cuda.synchronize()
    assert fm.device_status(dev) == 0
    assert int(workspace.view(torch.int32).abs().sum()) == 0, "workspace must be left zeroed"
    c_ref = F.gemm_reference(a.numpy(), _oracle_weight(w, qc, gs))
    return F.rel_frobenius(c.cpu().numpy().astype(np.float32), c_ref), c


def test_operands_are_bit_exact():
    """The fp16 values fed to the tensor cores equal the oracle's dequantised weights bit for bit."""
    dev = _dev()
    for (k, n, qc, gs) in [(256, 512, 256, 128), (128, 160, 32, 128), (192, 320, 64, -1), (256, 256, 256, -1), (512, 384, -1, 128)]:
        w = synth.make_weight_fp16(k, n, qc, seed=k + n)
        ww = fm.make_w46_weight(w, qc, gs).to(dev)
        dumped = fm.dump_operands(ww.B, ww.s, k, n, qc, gs).cpu().numpy()
        assert np.array_equal(dumped.view(np.uint16), _oracle_weight(w, qc, gs).view(np.uint16)), (k, n, qc, gs)


def test_every_fp6_code_dequantises_exactly():
    dev = _dev()
    k, n = 128, 64
    codes = (torch.arange(k * n, dtype=torch.int32) % 64).to(torch.uint8).reshape(k, n)
    s6 = torch.ones(n, dtype=torch.float16)
    B, s = fm.pack_b200(None, codes, None, s6, k, n, n, -1)
    dumped = fm.dump_operands(B.to(dev), s.to(dev), k, n, n, -1).cpu().numpy()
    assert np.array_equal(dumped.view(np.uint16), F.fp6_code_to_fp16_bits(codes.numpy()))


def test_one_hot_rows_reproduce_the_dequantised_weights():
    """With one-hot activation rows the GEMM returns rows of W: the kernel's zero-point correction,
    group scaling and FP6 exponent handling (subnormal codes included) must reproduce the oracle's
    dequantised weights exactly, since each output is a single product rounded once to fp16."""
    dev = _dev()
    for (k, n, qc, gs) in [(256, 512, 256, 128), (256, 384, 128, -1), (128, 256, 256, -1)]:
        w = synth.make_weight_fp16(k, n, qc, seed=3)
        w[:5, -3:] *= 0.01                                    # forces FP6 subnormals and zeros
        ww = fm.make_w46_weight(w, qc, gs, keep_dequantized=False).to(dev)
        w_deq = _oracle_weight(w, qc, gs)
        rows = [0, 1, 2, 3, 4, 7, 8, 15, 31, 32, 63, 64, 100, 127, k - 2, k - 1]
        a = torch.zeros((16, k), dtype=torch.float16)
        for i, kk in enumerate(rows):
            a[i, kk] = 1.0
        c = torch.zeros((16, n), dtype=torch.float16, device=dev)
        workspace = torch.zeros(n // 128 * 16, device=dev)
        fm.mul(a.to(dev), ww.B, c, ww.s, workspace, qc, group_size=gs, layout="b200")
        torch.cuda.synchronize()
        # exact equality of values (+0 and -0 compare equal)
        assert np.array_equal(c.cpu().numpy().astype(np.float32), w_deq[rows].astype(np.float32)), (k, n, qc, gs)


def test_config0_cpu_reference_case():
    err, _ = _run(16, 4096, 4096, 256, 128)
    assert err <= TOL, err


@pytest.mark.parametrize("m", [1, 2, 3, 4, 8, 12, 16, 24, 32, 48, 64, 118, 128, 152])
def test_tiles_int4_only(m):
    # test.py:183-190: N=512, K=1024, both tile hints (128x128 only up to 16 rows)
    for tk, tn in [(64, 256), (128, 128)]:
        if m > 16 and tk == 128:
            continue
        err, _ = _run(m, 1024, 512, -1, -1, tk, tn)
        assert err <= TOL, (m, tk, tn, err)


@pytest.mark.parametrize("k", [768, 832, 896, 64, 128, 192])
def test_k_not_multiple_of_pipeline_depth_and_tiny_k(k):
    # test.py:192-200
    err, _ = _run(16, k, 512, -1, -1, 64, 256)
    assert err <= TOL, (k, err)


@pytest.mark.parametrize("m", [1, 12, 16, 64, 65, 77, 152])
@pytest.mark.parametrize("n,k", [(256, 512), (512, 1024), (25600, 1024)])
def test_mixed(m, n, k):
    # test.py:229-237: 256 FP6 columns; N=256 is the all-FP6 case
    for gs in (-1, 128):
        err, _ = _run(m, k, n, 256, gs, 64, 256)
        assert err <= TOL, (m, n, k, gs, err)


@pytest.mark.parametrize("m,k,n,qc", [(1, 8192, 1280, 32), (16, 8192, 1280, 32), (16, 4096, 2048, 16),
                                      (5, 1024, 2688, 64), (16, 11008, 4096, 256), (32, 4096, 12288, 256)])
def test_sharded_and_llama_shapes(m, k, n, qc):
    # ragged strips: 1280-32 = 9.75 strips of INT4 columns, 16/32/64 FP6 columns
    tk, tn = (64, 256) if n % 256 == 0 else (128, 128)
    err, _ = _run(m, k, n, qc, 128, tk, tn)
    assert err <= TOL, (m, k, n, qc, err)


def test_few_ctas_and_repeatability():
    e1, c1 = _run(16, 1024, 1024, 256, 128, sms=3)
    e2, c2 = _run(16, 1024, 1024, 256, 128, sms=148)
    e3, c3 = _run(16, 1024, 1024, 256, 128, sms=148)
    assert max(e1, e2, e3) <= TOL
    # two issuing threads share an accumulator: the halves of a block may be added in either order, so two
    # runs agree to the last bit or two of fp16, not necessarily bit for bit
    ulp = torch.finfo(torch.float16).eps * c2.float().abs().clamp_min(2.0 ** -14)
    assert bool(((c2.float() - c3.float()).abs() <= 2 * ulp).all())
    # with ordered sums one thread issues a block's instructions: the split-K reduction and the sums are
    # deterministic, bit for bit
    previous = fm.set_ordered_sums(True)
    try:
        runs = [_run(16, 8192, 2048, 256, 128, sms=148)[1] for _ in range(3)]
        e4, _ = _run(16, 1024, 1024, 256, 128, sms=5)
    finally:
        fm.set_ordered_sums(previous)
    assert e4 <= TOL
    assert torch.equal(runs[0], runs[1]) and torch.equal(runs[1], runs[2]), "ordered sums must be deterministic"


def test_reference_layout_tensors_from_the_reference_generator(golden_dir):
    """mul() on tensors packed by the reference's own gen_mixed_weight (golden fixture) equals
    A @ W_ref with the reference's dequantised weights."""
    dev = _dev()
    g = np.load(os.path.join(golden_dir, "reference_generators.npz"))
    for name in ("int4", "fp6", "mixed"):
        k, n, qc = (int(x) for x in g[f"{name}_shape"])
        B = torch.from_numpy(g[f"{name}_packed"].copy()).to(dev)
        s = torch.from_numpy(g[f"{name}_s"].view(np.float16).copy()).to(dev)
        a = synth.make_activations(16, k, 7)
        c = torch.zeros((16, n), dtype=torch.float16, device=dev)
        workspace = torch.zeros(n // 128 * 16, device=dev)
        fp6_marlin.mul(a.to(dev), B, c, s, workspace, qc, 64, 256)
        torch.cuda.synchronize()
        c_ref = F.gemm_reference(a.numpy(), g[f"{name}_wref"].view(np.float16))
        assert F.rel_frobenius(c.cpu().numpy().astype(np.float32), c_ref) <= TOL, name


def test_errors_like_the_reference():
    # test.py:202-227
    dev = _dev()
    m, n, k = 16, 256, 64
    a = torch.randn((m, k), dtype=torch.half, device=dev)
    ww = fm.make_w46_weight(synth.make_weight_fp16(k, n, -1), -1, -1).to(dev)
    c = torch.zeros((m, n), dtype=torch.half, device=dev)
    workspace = torch.zeros(n // 128, device=dev)
    for tk, tn in [(128, 128), (256, 256)]:
        with pytest.raises(RuntimeError):
            fm.mul(a, ww.B, c, ww.s, torch.zeros(n // 128 * 16, device=dev), -1, tk, tn, -1, layout="b200")
    with pytest.raises(RuntimeError, match="workspace"):
        fm.mul(a, ww.B, c, ww.s, workspace, -1, 64, 256, -1, layout="b200")
    with pytest.raises(RuntimeError):
        fm.mul(a.cpu(), ww.B, c, ww.s, workspace, layout="b200")     # no CPU path
    # zero-sized problems are silent no-ops (fp6_marlin_cuda_kernel.cu:906-907)
    fm.mul(a[:0], ww.B, c[:0], ww.s, torch.zeros(32, device=dev), -1, 64, 256, layout="b200")


def test_full_size_against_fp32_matmul_of_dumped_operands():
    """K = N = 8192 (the benchmark layer): the operands the kernel uses are dumped, checked equal to
    the product-side dequantised weights, and the result is compared with an fp32 matmul of them."""
    dev = _dev()
    k = n = 8192
    layer = synth.make_layer(k, n, 256, 128, seed=1)
    ww = layer.to(dev)
    dumped = fm.dump_operands(ww.B, ww.s, k, n, 256, 128)
    assert torch.equal(dumped, ww.w_deq)
    for m in (1, 16, 64):
        a = synth.make_activations(m, k, m).to(dev)
        c = torch.zeros((m, n), dtype=torch.float16, device=dev)
        workspace = torch.zeros(n // 128 * 16, device=dev)
        fm.mul(a, ww.B, c, ww.s, workspace, 256, group_size=128, layout="b200")
        c_ref = a.float() @ dumped.float()
        err = (torch.linalg.norm(c.float() - c_ref) / torch.linalg.norm(c_ref)).item()
        assert err <= TOL, (m, err)
    assert fm.device_status(dev) == 0


@pytest.mark.gpu
def test_launch_overlap_keeps_dependent_chains_exact():
    """With programmatic dependent launch on, a GEMM starts while its predecessor drains; a chain
    C1 = A W1, C2 = C1 W2, ... (each GEMM reads what the previous one wrote, all share one scratch and
    one output buffer per parity) must give bit-identical results to the same chain without overlap."""
    dev = _dev()
    k = n = 2048
    layers = [synth.make_layer(k, n, 256, 128, seed=20 + i, keep_dequantized=False).to(dev) for i in range(4)]
    a0 = (synth.make_activations(16, k, 9) * 0.05).to(dev)
    workspace = torch.zeros(n // 128 * 16, dtype=torch.int32, device=dev)

    def chain():
        bufs = [torch.zeros((16, n), dtype=torch.float16, device=dev) for _ in range(2)]
        x = a0
        outs = []
        for rep in range(3):
            for i, w in enumerate(layers):
                y = bufs[(rep * len(layers) + i) % 2]
                fm.mul(x, w.B, y, w.s, workspace, 256, group_size=128, layout="b200")
                x = y
                outs.append((y.float().abs().sum() * 0 + y.float().square().sum()).clone())
            x = (x * 0.01).clone()      # keep the magnitudes in range between repetitions
        torch.cuda.synchronize()
        return torch.stack(outs), x.clone()

    previous = fm.set_launch_overlap(False)
    ordered = fm.set_ordered_sums(True)         # bit-identical sums from run to run, so that the chains can be compared exactly
    try:
        ref_sums, ref_last = chain()
        fm.set_launch_overlap(True)
        got_sums, got_last = chain()
    finally:
        fm.set_launch_overlap(previous)
        fm.set_ordered_sums(ordered)
    assert torch.isfinite(ref_last.float()).all()
    assert torch.equal(ref_sums, got_sums)
    assert torch.equal(ref_last, got_last)
    assert fm.device_status(dev) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("m", [17, 33, 100, 129, 256, 257, 300, 700])
def test_wide_tiles_and_passes(m):
    """More than 16 rows: MMA tiles of 32/64/128/256 rows, ragged last tile, several passes of 256 rows."""
    for (k, n, qc, gs) in [(1024, 2048, 256, 128), (512, 1280, 256, -1), (2048, 768, -1, 128)]:
        err, _ = _run(m, k, n, qc, gs, 64, 256, seed=m)
        assert err <= TOL, (m, k, n, qc, gs, err)


@pytest.mark.gpu
@pytest.mark.parametrize("m", [12, 24, 60, 100, 200, 600])
def test_ordered_sums_instances_against_the_oracle(m):
    """The "ordered sums" instances of both kernels (one issuing thread per accumulator tile) are kernels of their
    own: every tile width against the oracle, and two runs bit for bit."""
    previous = fm.set_ordered_sums(True)
    try:
        for (k, n, qc, gs) in [(1024, 2048, 256, 128), (2048, 768, -1, 128), (8192, 1024, 256, 128)]:
            err, c1 = _run(m, k, n, qc, gs, 64, 256, seed=m)
            assert err <= TOL, (m, k, n, qc, gs, err)
            _, c2 = _run(m, k, n, qc, gs, 64, 256, seed=m)
            assert torch.equal(c1, c2), (m, k, n, qc, gs)
    finally:
        fm.set_ordered_sums(previous)


@pytest.mark.gpu
def test_wide_one_hot_rows_reproduce_scaled_weights_exactly():
    """With group scales the wide kernel feeds fp16((q - 8) * s_g) to the tensor cores: one-hot rows of A
    must return exactly the oracle's dequantised weights (the fp32 sum has a single term)."""
    dev = _dev()
    k, n, qc, gs = 256, 512, 256, 128
    w = synth.make_weight_fp16(k, n, qc, seed=5)
    ww = fm.make_w46_weight(w, qc, gs, keep_dequantized=False).to(dev)
    a = torch.eye(k, dtype=torch.float16)[:200].contiguous().to(dev)       # rows 0..199 of the identity
    c = torch.zeros((200, n), dtype=torch.float16, device=dev)
    workspace = torch.zeros(max(n // 128 * 16, 16), dtype=torch.int32, device=dev)
    fm.mul(a, ww.B, c, ww.s, workspace, qc, 64, 256, group_size=gs, layout="b200")
    torch.cuda.synchronize()
    expect = _oracle_weight(w, qc, gs)[:200]
    assert np.array_equal(c.cpu().numpy().view(np.uint16), expect.view(np.uint16))


@pytest.mark.gpu
def test_wide_long_k_and_split_strips():
    """K = 8192 with few strips: every strip is shared by several CTAs (tagged split-K slots of 256 rows)."""
    err, _ = _run(256, 8192, 1024, 256, 128, 64, 256, seed=3)
    assert err <= TOL, err
    err, _ = _run(40, 8192, 512, -1, 128, 64, 256, seed=4)
    assert err <= TOL, err


@pytest.mark.gpu
def test_w46_linear_forward_matches_dequantised_matmul():
    dev = _dev()
    torch.manual_seed(1)
    out_f, in_f, qc = 768, 512, 256
    w = torch.randn(out_f, in_f) * 0.02
    w[torch.randperm(out_f)[:qc]] *= 8
    bias = torch.randn(out_f).half()
    x = torch.randn(3, 5, in_f).half()
    for restore in (True, False):
        layer = fm.W46Linear(w.half(), quant_cols=qc, group_size=128, bias=bias, restore_order=restore).to(dev)
        y = layer(x.to(dev)).float().cpu()
        perm = layer.output_permutation.cpu()
        w_kn = w.half().t().contiguous()[:, perm]
        ref = F.gemm_reference(x.reshape(-1, in_f).numpy(), _oracle_weight(w_kn, qc, 128))       # columns in mul's order
        ref = torch.from_numpy(ref) + bias.float()[perm]
        if restore:
            ref = ref[:, layer.inverse_permutation.cpu()]
        err = (torch.linalg.norm(y.reshape(-1, out_f) - ref) / torch.linalg.norm(ref)).item()
        assert err <= 2 * TOL, (restore, err)        # the bias is added in fp16 after the GEMM's own rounding


@pytest.mark.gpu
def test_gpu_weight_preparation_matches_host_bytes():
    """Quantise + cast + pack on the GPU gives the same packed words and scales as the host path."""
    dev = _dev()
    for (k, n, qc, gs) in [(256, 512, 256, 128), (384, 1280 + 32, 32, 128), (192, 320, 64, -1), (256, 256, 256, -1), (512, 384, -1, 128)]:
        w = synth.make_weight_fp16(k, n, qc, seed=k + n)
        host = fm.make_w46_weight(w, qc, gs)
        gpu = fm.make_w46_weight(w, qc, gs, quant_device=dev)
        assert gpu.B.device.type == "cuda"
        assert torch.equal(gpu.B.cpu(), host.B), (k, n, qc, gs)
        assert torch.equal(gpu.s.cpu().view(torch.int16), host.s.view(torch.int16)), (k, n, qc, gs)
        assert torch.equal(gpu.w_deq.cpu().view(torch.int16), host.w_deq.view(torch.int16)), (k, n, qc, gs)


@pytest.mark.gpu
def test_gpu_fp6_cast_matches_host_on_every_in_range_half():
    dev = _dev()
    bits = torch.arange(0, 1 << 16, dtype=torch.int32).to(torch.int16)
    vals = bits.view(torch.float16)
    mag = vals.abs().float()
    ok = (mag == 0) | ((mag >= 0.0625) & (mag <= 28.0))
    x = vals[ok].contiguous()
    assert torch.equal(fm.encode_fp6_gpu(x.to(dev)).cpu(), fm.encode_fp6(x))
    with pytest.raises(ValueError):
        fm.encode_fp6_gpu(torch.tensor([0.01, 1.0], dtype=torch.float16, device=dev))
    with pytest.raises(ValueError):
        fm.encode_fp6_gpu(torch.tensor([29.0], dtype=torch.float16, device=dev))


@pytest.mark.gpu
@pytest.mark.parametrize("m,k,n,qc,n_total,col4,col6", [
    (16, 512, 512, 128, 2048, 384, 1536 + 128),
    (48, 512, 512, 128, 2048, 384, 1536 + 128),
    (48, 512, 512, 128, 2048, 388, 1536 + 132),       # up to 128 rows: C leaves as 8-byte stores, these outputs as 2-byte stores
    (100, 2048, 512, 128, 2048, 384, 1536 + 128),     # 128-row tile, strips shared by two CTAs and reduced by eight groups
    (100, 2048, 512, 128, 2048, 388, 1536 + 132),
    (30, 2048, 512, 128, 2048, 388, 1536 + 132),
    (300, 512, 512, 128, 2048, 384, 1536 + 128),      # the kernel for more than 128 rows, 16-byte row stores
    (300, 512, 512, 128, 2048, 388, 1536 + 132),      # column bases off the 16-byte grid: 2-byte stores
    (200, 1024, 1248 + 32, 32, 4096, 1248, 3000),     # ragged strips (9.75 INT4 strips, 32 FP6 columns)
    (2300, 16384, 256, 64, 512, 64, 320),             # K = 16384: two launches (2048 rows and a ragged tail)
])
def test_mul_scatter_places_a_shard_in_full_width_outputs(m, k, n, qc, n_total, col4, col6):
    """fp6m_mul_scatter (the GEMM whose epilogue is the all-gather): with two local buffers standing in for two
    ranks' outputs, the shard's INT4 and FP6 columns land at their places among the layer's columns and the
    values are those of the plain GEMM."""
    import ctypes
    from fp6_marlin_b200 import _lib, api
    dev = _dev()
    gs = 128
    w = synth.make_weight_fp16(k, n, qc, seed=11)
    ww = fm.make_w46_weight(w, qc, gs, keep_dequantized=False).to(dev)
    a = synth.make_activations(m, k, 11).to(dev)
    c = torch.zeros((m, n), dtype=torch.float16, device=dev)
    workspace = torch.zeros(max(n // 128 * 16, 64), dtype=torch.int32, device=dev)
    ordered = fm.set_ordered_sums(True)          # both GEMMs add in one fixed order: comparable bit for bit
    try:
        fm.mul(a, ww.B, c, ww.s, workspace, qc, group_size=gs, layout="b200")
        outs = [torch.full((m, n_total), -7.0, dtype=torch.float16, device=dev) for _ in range(2)]
        table = (ctypes.c_void_p * 2)(*[o.data_ptr() for o in outs])
        _, scratch, status = api._device_buffers(dev, (m, n, k, qc))
        rc = _lib.lib.fp6m_mul_scatter(a.data_ptr(), ww.B.data_ptr(), table, 2, n_total, col4, col6, ww.s.data_ptr(), m, n, k,
                                       workspace.data_ptr(), workspace.numel() * 4, scratch.data_ptr(), scratch.numel(), dev.index or 0,
                                       torch.cuda.current_stream(dev).cuda_stream, -1, -1, -1, 16, qc, gs, _lib.LAYOUT_B200,
                                       status.data_ptr())
        assert rc == _lib.OK
        torch.cuda.synchronize()
    finally:
        fm.set_ordered_sums(ordered)
    c_ref = F.gemm_reference(a.cpu().numpy(), _oracle_weight(w, qc, gs))
    assert F.rel_frobenius(c.cpu().numpy().astype(np.float32), c_ref) <= TOL
    for o in outs:
        assert torch.equal(o[:, col4:col4 + n - qc], c[:, : n - qc])
        assert torch.equal(o[:, col6:col6 + qc], c[:, n - qc:])
        untouched = torch.ones(n_total, dtype=torch.bool, device=dev)
        untouched[col4:col4 + n - qc] = False
        untouched[col6:col6 + qc] = False
        assert bool((o[:, untouched] == -7.0).all())
    assert fm.device_status(dev) == 0

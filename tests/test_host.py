"""CPU tests of the product's host side: the reference-compatible quantize / prepacking /
dequantize, the b200 layout packers, the reference->b200 converter, the stripe schedule, and the
C ABI surface.  No GPU compute is called here."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import fp6_marlin_b200 as fm
from fp6_marlin_b200 import _lib
from oracle import formats as F


def _h(bits):
    return np.asarray(bits).view(np.float16)


# ---------------------------------------------------------------- C ABI surface
def test_library_exports_every_declared_symbol():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    header = open(os.path.join(root, "include", "fp6m.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(fp6m_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(raw, name), f"{name} is declared in include/fp6m.h but not exported"
    assert declared == set(_lib.SIGNATURES), "python binding and header disagree"
    assert "sm_100a" in _lib.lib.fp6m_version().decode()


def test_drop_in_module_surface():
    import inspect

    import fp6_marlin
    for name in ("prepacking", "quantize", "dequantize", "mul"):
        assert callable(getattr(fp6_marlin, name))
    sig = inspect.signature(fp6_marlin.mul)
    names = list(sig.parameters)
    assert names[:10] == ["A", "B", "C", "s", "workspace", "quant_cols", "thread_k", "thread_n", "sms", "max_par"]
    defaults = [sig.parameters[n].default for n in names[5:10]]
    assert defaults == [-1, -1, -1, -1, 16]          # fp6_marlin/__init__.py:39


def test_extension_module_names_of_the_reference():
    """``import fp6_marlin_cuda`` / ``import fp6_marlin_cpu`` (the reference's two extension modules,
    setup.py:38,48; bound names pybind.cpp:89-94 and fp6_marlin_cuda.cpp:125-127) resolve to this library."""
    import inspect

    import fp6_marlin_cpu
    import fp6_marlin_cuda
    for name in ("quantization_cpu", "prepacking_cpu", "dequantization_cpu"):
        assert callable(getattr(fp6_marlin_cpu, name))
    sig = inspect.signature(fp6_marlin_cuda.mul)
    assert list(sig.parameters) == ["A", "B", "C", "s", "workspace", "quant_cols", "thread_k", "thread_n", "sms", "max_par"]
    assert sig.parameters["max_par"].default == 8     # fp6_marlin_cuda.cpp:57
    x = torch.zeros((256, 256), dtype=torch.float16)
    x[0, 0] = 1.5
    stream = fp6_marlin_cpu.quantization_cpu(x)
    assert stream.shape == (256, 48) and stream.dtype == torch.int32
    assert fp6_marlin_cpu.prepacking_cpu(stream).shape == (24, 512)
    back = fp6_marlin_cpu.dequantization_cpu(stream, torch.ones(256, dtype=torch.float16))
    assert float(back[0, 0]) == 1.5 and float(back.abs().sum()) == 1.5


# ---------------------------------------------------------------- reference-compatible host functions
def test_host_functions_match_reference_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "fp6_host_256x256.npz"))
    w = torch.from_numpy(_h(g["w"]).copy())
    s = torch.from_numpy(_h(g["s"]).copy())
    q = fm.quantize(w)
    assert q.dtype == torch.int32 and tuple(q.shape) == (256, 48)
    assert np.array_equal(q.numpy(), g["quantized"])
    p = fm.prepacking(q)
    assert tuple(p.shape) == (24, 512) and np.array_equal(p.numpy(), g["prepacked"])
    d = fm.dequantize(q, s)
    assert tuple(d.shape) == (256, 256) and np.array_equal(d.numpy().view(np.uint16), g["dequantized"])


def test_host_functions_match_oracle_rectangular():
    rng = np.random.default_rng(5)
    w = rng.uniform(-28, 28, size=(512, 256)).astype(np.float16)
    w = np.where(np.abs(w) < np.float16(0.0625), np.float16(0), w).astype(np.float16)
    q = fm.quantize(torch.from_numpy(w))
    assert tuple(q.shape) == (256, 96)
    assert np.array_equal(q.numpy(), F.fp6_quantize(w))
    s = rng.uniform(0.01, 1.0, size=256).astype(np.float16)
    assert np.array_equal(fm.dequantize(q, torch.from_numpy(s)).numpy().view(np.uint16),
                          F.fp6_dequant(q.numpy(), s).view(np.uint16))
    assert np.array_equal(fm.prepacking(q).numpy(), F.fp6_prepack_reference(q.numpy()))


def test_quantize_errors():
    with pytest.raises(ValueError, match="float16"):
        fm.quantize(torch.zeros(256, 256, dtype=torch.float32))
    with pytest.raises(ValueError, match="out of range"):
        fm.quantize(torch.full((256, 256), 30.0, dtype=torch.float16))
    with pytest.raises(ValueError, match="out of range"):
        fm.quantize(torch.full((256, 256), 0.01, dtype=torch.float16))
    with pytest.raises(ValueError):
        fm.quantize(torch.zeros(100, 256, dtype=torch.float16))      # the reference aborts here
    with pytest.raises(ValueError):
        fm.prepacking(torch.zeros(64, 48, dtype=torch.int32))
    # zeros are fine
    assert int(fm.quantize(torch.zeros(256, 256, dtype=torch.float16)).abs().sum()) == 0


def test_encode_every_code():
    codes = torch.arange(64, dtype=torch.uint8)
    vals = fm.decode_fp6(codes)
    keep = (codes & 0x1F) != 0                                   # +-0 both encode to their own sign
    assert torch.equal(fm.encode_fp6(vals)[keep], codes[keep])
    assert np.array_equal(vals.numpy().view(np.uint16), F.fp6_code_to_fp16_bits(codes.numpy()))


# ---------------------------------------------------------------- quantisers against the oracle
@pytest.mark.parametrize("group_size", [-1, 128])
def test_int4_quantiser_matches_oracle(group_size):
    torch.manual_seed(2)
    w = (torch.randn(256, 96) * 0.02).half()
    w[:, 5] = 0                                                  # an all-zero column / group
    q, s, deq = fm.quantize_int4(w, group_size)
    if group_size > 0:
        qo, so, do = F.int4_quantize_group(w.numpy(), group_size)
        assert np.array_equal(q.numpy(), qo) and np.array_equal(s.numpy().view(np.uint16), so.view(np.uint16))
        assert np.array_equal(deq.numpy().view(np.uint16), do.view(np.uint16))
    else:
        w[:, 5] = 0.01                                           # per-channel rule divides by the scale
        q, s, deq = fm.quantize_int4(w, group_size)
        qo, so, do = F.int4_quantize_per_channel(w.numpy())
        assert np.array_equal(q.numpy(), qo) and np.array_equal(s.numpy().view(np.uint16), so.view(np.uint16))
        assert np.array_equal(deq.numpy().view(np.uint16), do.view(np.uint16))
    assert np.array_equal(F.int4_dequant(q.numpy(), s.numpy(), group_size).view(np.uint16), deq.numpy().view(np.uint16))


def test_fp6_quantiser_matches_oracle():
    torch.manual_seed(4)
    w = (torch.randn(128, 64) * 0.3).half()
    c, s, deq = fm.quantize_fp6(w)
    co, so, do = F.fp6_codes_and_dequant(w.numpy())
    assert np.array_equal(c.numpy(), co) and np.array_equal(s.numpy().view(np.uint16), so.view(np.uint16))
    assert np.array_equal(deq.numpy().view(np.uint16), do.view(np.uint16))


# ---------------------------------------------------------------- b200 layout
B200_CASES = [(256, 512, 256, 128), (128, 160, 32, 128), (64, 96, 16, -1), (192, 64, 64, -1),
              (256, 128, -1, 128), (256, 288, 288, -1), (384, 1280, 32, 128), (64, 8, -1, -1), (200, 264, 8, -1)]


@pytest.mark.parametrize("k,n,qc,gs", B200_CASES)
def test_b200_pack_unpack_round_trip(k, n, qc, gs):
    rng = np.random.default_rng(k + n)
    nq = max(qc, 0)
    groups = (k + 127) // 128 if gs > 0 else 1
    q4 = torch.from_numpy(rng.integers(0, 16, size=(k, n - nq), dtype=np.uint8))
    c6 = torch.from_numpy(rng.integers(0, 64, size=(k, nq), dtype=np.uint8))
    s4 = torch.from_numpy(rng.standard_normal((groups, n - nq)).astype(np.float16))
    s6 = torch.from_numpy(rng.standard_normal(nq).astype(np.float16))
    B, s = fm.pack_b200(q4 if n - nq else None, c6 if nq else None, s4 if n - nq else None, s6 if nq else None, k, n, qc, gs)
    words, nscales = fm.b200_sizes(k, n, qc, gs)
    assert B.numel() == words and s.numel() == nscales
    r4, r6, rs4, rs6 = fm.unpack_b200(B, s, k, n, qc, gs)
    assert torch.equal(r4, q4) and torch.equal(r6, c6)
    assert torch.equal(rs4, s4) and torch.equal(rs6, s6)


def test_b200_sizes_equal_reference_sizes_for_aligned_shapes():
    # same bits, different tiling: for shapes the reference supports the byte counts agree
    for (k, n, qc) in [(4096, 4096, 256), (8192, 8192, 256), (1024, 512, -1), (512, 256, 256)]:
        nq = max(qc, 0)
        words, nscales = fm.b200_sizes(k, n, qc, -1)
        assert words * 4 == k * (n - nq) // 2 + k * nq * 3 // 4
        assert nscales == n


def test_b200_word_layout_by_hand():
    """One INT4 word and one FP6 word decoded by the rules in fp6m_layout.h."""
    k, n = 128, 64
    q4 = torch.zeros((k, 32), dtype=torch.uint8) + 8
    c6 = torch.zeros((k, 32), dtype=torch.uint8)
    # column 9, rows 104..111 = unit 1 (rows 64..127), word w8 = 5
    q4[104:112, 9] = torch.arange(1, 9, dtype=torch.uint8)
    c6[104:112, 9] = torch.tensor([0b100001, 0b010010, 0b110011, 0b000100, 0b101111, 0b011010, 0b111001, 0b001000], dtype=torch.uint8)
    B, s = fm.pack_b200(q4, c6, torch.ones(1, 32).half(), (torch.arange(32) + 1).half(), k, n, 32, -1)
    raw = B.numpy().view(np.uint8)
    nq, unit, c, w8 = 1, 1, 9, 5
    off = unit * nq * 1024 + c * 32 + 16 * ((w8 >> 2) ^ ((c >> 2) & 1)) + 4 * (w8 & 3)
    word = int(raw[off:off + 4].view(np.uint32)[0])
    assert [(word >> (4 * p)) & 15 for p in range(8)] == [1, 3, 5, 7, 2, 4, 6, 8]     # rows i = 0,2,4,6,1,3,5,7
    fp6_base = 2 * nq * 1024 + unit * nq * 1536                # INT4 region (two units), then FP6 units
    four = int(raw[fp6_base + c * 32 + 16 * ((w8 >> 2) ^ ((c >> 2) & 1)) + 4 * (w8 & 3):][:4].view(np.uint32)[0])
    two = int(raw[fp6_base + nq * 1024 + c * 16 + 4 * (w8 >> 1):][:4].view(np.uint32)[0])
    codes = c6[104:112, 9].tolist()
    for i in range(8):
        b, js = i % 4, 2 * (w8 & 1) + i // 4
        lo = (four >> (8 * b + 4 * (i // 4))) & 15
        rot = ((two << (2 * js)) | (two >> (32 - 2 * js))) & 0xFFFFFFFF if js else two
        hi = (rot >> (8 * b)) & 0x90
        assert lo == codes[i] & 15
        assert hi == ((codes[i] >> 5) << 7 | ((codes[i] >> 4) & 1) << 4)
    # scales are in plain column order: INT4 scales (padded to 32), then FP6 scales
    assert s.numel() == 64 and float(s[32 + 9]) == 10.0


@pytest.mark.parametrize("name", ["int4", "fp6", "mixed"])
def test_repack_from_reference_golden(golden_dir, name):
    """Tensors produced by the reference's own generators -> b200 layout -> logical codes equal the
    codes the oracle derives from the same weights."""
    g = np.load(os.path.join(golden_dir, "reference_generators.npz"))
    k, n, qc = (int(x) for x in g[f"{name}_shape"])
    nq = max(qc, 0)
    B, s = fm.repack_from_reference(torch.from_numpy(g[f"{name}_packed"].copy()),
                                    torch.from_numpy(_h(g[f"{name}_s"]).copy()), k, n, qc)
    q4, c6, s4, s6 = fm.unpack_b200(B, s, k, n, qc, -1)
    w = _h(g[f"{name}_w"])
    wref = _h(g[f"{name}_wref"])
    if n - nq:
        qo, so, do = F.int4_quantize_per_channel(w[:, : n - nq])
        assert np.array_equal(q4.numpy(), qo) and np.array_equal(s4.numpy().reshape(-1).view(np.uint16), so.view(np.uint16))
        assert np.array_equal(F.int4_dequant(q4.numpy(), s4.numpy().reshape(-1)).view(np.uint16), wref[:, : n - nq].view(np.uint16))
    if nq:
        vals = _h(F.fp6_code_to_fp16_bits(c6.numpy())).astype(np.float32)
        deq = (vals * s6.numpy().astype(np.float32).reshape(1, -1)).astype(np.float16)
        assert np.array_equal(deq.view(np.uint16), wref[:, n - nq:].view(np.uint16))


# ---------------------------------------------------------------- stripe schedule
@pytest.mark.parametrize("k,n,qc,ctas", [(8192, 8192, 256, 148), (4096, 4096, 256, 148), (11008, 4096, 256, 148),
                                         (4096, 22016, 256, 148), (64, 256, -1, 148), (512, 256, 256, 148),
                                         (8192, 1280, 32, 148), (1024, 25600, 256, 132), (256, 512, 256, 1),
                                         (16384, 16384, 512, 296)])
def test_schedule_covers_every_unit_once(k, n, qc, ctas):
    """Units are 64 rows of one 128-column strip; every unit belongs to exactly one CTA and the
    cost per CTA (8 per INT4 unit, 11 per FP6 unit) is balanced to within one unit - plus the one segment
    (16 cost units) by which CTAs that reduce a strip at their end are given less than the others."""
    bounds, total = fm.schedule(k, n, qc, 128 if k % 128 == 0 else -1, ctas)
    nq = max(qc, 0)
    s4 = -(-(n - nq) // 128)
    strips = s4 + -(-nq // 128)
    ups = 2 * -(-k // 128)
    assert total == strips * ups
    assert bounds[0] == 0 and bounds[-1] == total and len(bounds) == ctas + 1
    assert all(b1 >= b0 for b0, b1 in zip(bounds, bounds[1:]))

    def cost(unit):
        return 8 if unit // ups < s4 else 11
    costs = np.array([cost(u) for u in range(total)], dtype=np.int64)
    csum = np.concatenate([[0], np.cumsum(costs)])
    per_cta = np.array([csum[b1] - csum[b0] for b0, b1 in zip(bounds, bounds[1:])])
    assert per_cta.sum() == costs.sum()
    assert per_cta.max() <= costs.sum() / ctas + 16 + 11 + 1e-9
    if ctas > 1 and total // ctas >= 16:
        assert per_cta.min() >= costs.sum() / ctas - 16 - 11 - 1e-9


def test_w46_linear_bookkeeping():
    """The linear wrapper moves the largest-magnitude output features to the FP6 end and remembers how."""
    torch.manual_seed(0)
    out_f, in_f, qc = 512, 256, 256
    w = torch.randn(out_f, in_f) * 0.02
    hot = torch.randperm(out_f)[:qc]
    w[hot] *= 8
    layer = fm.W46Linear(w.half(), quant_cols=qc, group_size=128)
    perm, inv = layer.output_permutation, layer.inverse_permutation
    assert sorted(perm.tolist()) == list(range(out_f))
    assert torch.equal(perm[inv], torch.arange(out_f)) and torch.equal(inv[perm], torch.arange(out_f))
    assert set(perm[out_f - qc:].tolist()) == set(hot.tolist())            # the outliers are the FP6 columns
    assert perm[: out_f - qc].tolist() == sorted(perm[: out_f - qc].tolist())   # the others keep their order
    nwords, nscales = fm.b200_sizes(in_f, out_f, qc, 128)
    assert layer.B.numel() == nwords and layer.s.numel() == nscales
    assert "fp6_columns=256" in repr(layer)


def test_launch_plan_and_scratch_sizes():
    """How the host cuts M rows into launches (the reference's dispatcher loops over batches of rows as well,
    fp6_marlin_cuda_kernel.cu:917-948): one launch of the kernel for up to 128 rows; 129 to 256 rows as two launches
    of it on a layer with at most 48 blocks per CTA, else one 256-row tile of the other kernel; more rows in launches
    whose activations stay within 64 MB.  The scratch size asked for without a device covers either plan."""
    sms = 148
    assert fm.launch_plan(0, 8192, 8192, 256, sms) == (0, False)
    for m in (1, 16, 17, 64, 128):
        assert fm.launch_plan(m, 8192, 8192, 256, sms) == (1, False)
    for m in (129, 200, 256):
        assert fm.launch_plan(m, 8192, 8192, 256, sms) == (2, False)        # 64 strips x 64 blocks = 28 per CTA
        assert fm.launch_plan(m, 16384, 16384, 256, sms) == (1, True)       # 128 x 128 blocks = 111 per CTA
    assert fm.launch_plan(257, 8192, 8192, 256, sms) == (1, True)
    assert fm.launch_plan(8192, 8192, 8192, 256, sms) == (2, True)          # 16 tiles of 256 rows x 16 KB per row = 64 MB
    assert fm.launch_plan(8192, 16384, 16384, 256, sms) == (4, True)        # K = 16384: eight tiles per launch
    assert fm.launch_plan(8192, 2048, 16384, 32, sms) == (4, True)
    need = _lib.lib.fp6m_mul_scratch_bytes
    for shape in ((200, 8192, 8192, 256), (200, 16384, 16384, 256), (256, 4096, 4096, -1)):
        assert need(*shape, -1) >= need(*shape, sms)
        assert need(*shape, -1) >= need(*shape, 8)                           # a device with few SMs takes the other plan
    assert need(0, 0, 0, 0, -1) >= need(8192, 16384, 16384, 256, sms)
    assert need(128, 8192, 8192, 256, sms) >= need(16, 8192, 8192, 256, sms)

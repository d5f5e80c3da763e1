"""TEST INFRASTRUCTURE ONLY (the oracle).  Nothing in the product path may import this module;
only tests/, the smoke check and the CPU-baseline leg of the benchmark use it, as the checker.

NumPy restatement of the reference's weight formats and of its host-side algorithms for the
W(4&6)A16 GEMM path.  Every function names the reference lines it restates.  The restatement is
pinned two ways (tests/test_oracle.py): against the reference's own host code compiled from its
sources (oracle/_ref, built by oracle/build_ref.py) wherever that library is present, and against
the golden vectors under tests/golden/ that were generated from that library.

Conventions: fp16 data travels as ``np.float16`` arrays or as their ``uint16`` bit patterns;
logical weights are ``W[k, n]`` (k = reduction index, n = output column); a "stream" is the
reference's dense 6-bit packing, 4 codes in 3 bytes.
"""
from __future__ import annotations

import numpy as np

FP6_MAX = 28.0        # weight_quant.cpp:43
FP6_MIN = 0.0625      # weight_quant.cpp:40

# --------------------------------------------------------------------------------------------
# FP6 E3M2: cast, dense stream, dequantisation
# --------------------------------------------------------------------------------------------


def fp6_encode(w: np.ndarray) -> np.ndarray:
    """fp16 -> 6-bit codes ``s eee mm`` (uint8), truncating the mantissa.

    Restates ``cast_fp16_fp6`` (fp6_marlin/weight_quant.cpp:27-91): bias-3 exponent, exponent 7 is
    an ordinary value, fp16 subnormals become 0, FP6 subnormals are made by shifting the mantissa
    with its implicit one to the right (no rounding), and a value with ``0 < |x| < 0.0625`` or
    ``|x| > 28`` raises (the reference throws std::invalid_argument, weight_quant.cpp:48-53).
    """
    w = np.ascontiguousarray(w)
    if w.dtype != np.float16:
        raise ValueError("Input tensor should be of type float16.")
    a = np.abs(w.astype(np.float32))
    if np.any(((a != 0) & (a < FP6_MIN)) | (a > FP6_MAX)) or np.any(np.isnan(a)):
        raise ValueError("Input value out of range for FP6.")
    bits = w.view(np.uint16).astype(np.int32)
    sign = bits >> 15
    exp = (bits & 0x7FFF) >> 10
    mant = bits & 0x3FF
    new_mant = mant >> 8
    new_exp = exp - 15 + 3
    target = exp - 15
    sub = target < -2                               # below the smallest normal FP6 exponent
    shift = np.clip(-2 - target, 0, 31)
    new_mant = np.where(sub, (new_mant | 4) >> shift, new_mant)
    new_exp = np.where(sub, 0, new_exp)
    zero = exp == 0                                 # fp16 subnormal or zero
    new_mant = np.where(zero, 0, new_mant)
    new_exp = np.where(zero, 0, new_exp)
    return ((sign << 5) | (new_exp << 2) | new_mant).astype(np.uint8)


def fp6_pack_stream(codes: np.ndarray) -> np.ndarray:
    """6-bit codes (..., 4m) -> dense bytes (..., 3m): ``[a5..a0 b5 b4][b3..b0 c5..c2][c1 c0 d5..d0]``
    (fp6_marlin/weight_quant.cpp:93-95)."""
    c = codes.astype(np.uint32).reshape(*codes.shape[:-1], -1, 4)
    b0 = (c[..., 0] << 2) | (c[..., 1] >> 4)
    b1 = ((c[..., 1] & 0xF) << 4) | (c[..., 2] >> 2)
    b2 = ((c[..., 2] & 0x3) << 6) | c[..., 3]
    out = np.stack([b0, b1, b2], axis=-1).astype(np.uint8)
    return out.reshape(*codes.shape[:-1], -1)


def fp6_unpack_stream(stream: np.ndarray) -> np.ndarray:
    """Inverse of :func:`fp6_pack_stream`; the bit positions are the ones
    ``Extract_6_Bits_To_A_Byte`` reads (fp6_marlin/weight_prepacking.cpp:40-54, 192-197)."""
    b = stream.astype(np.uint32).reshape(*stream.shape[:-1], -1, 3)
    c0 = b[..., 0] >> 2
    c1 = ((b[..., 0] & 0x3) << 4) | (b[..., 1] >> 4)
    c2 = ((b[..., 1] & 0xF) << 2) | (b[..., 2] >> 6)
    c3 = b[..., 2] & 0x3F
    out = np.stack([c0, c1, c2, c3], axis=-1).astype(np.uint8)
    return out.reshape(*stream.shape[:-1], -1)


def fp6_quantize(w: np.ndarray) -> np.ndarray:
    """``quantize`` of the reference: (a, b) fp16 -> (b, a*3/16) int32.

    Restates ``weight_quantization_cpu`` (fp6_marlin/pybind.cpp:42-59) together with
    ``weight_prepacking_fp16_to_fp6`` (weight_quant.cpp:106-124).  The row-major MEMORY of the
    input is packed as it lies: the transpose at pybind.cpp:52 is a view whose data pointer is the
    original one, so only the shape label of the result is transposed.
    """
    if w.dtype != np.float16:
        raise ValueError("Input tensor should be of type float16.")
    a, b = w.shape
    if a % 256 or b % 256:
        raise ValueError("quantize: both dimensions must be multiples of 256")
    flat = np.ascontiguousarray(w).reshape(-1)
    stream = fp6_pack_stream(fp6_encode(flat))
    return stream.view(np.int32).reshape(b, a * 3 // 16)


def fp6_code_to_fp16_bits(codes: np.ndarray) -> np.ndarray:
    """Exact E3M2 value of each code as fp16 bits.

    Restates the bit path of ``dequantMatrix_fp6_to_fp16`` (weight_prepacking.cpp:199-212): the code
    is placed as ``s 00eee mm 0...`` in an fp16 and multiplied by 2**12 (exact, subnormals included).
    """
    c = codes.astype(np.uint16)
    raw = ((c & 0x20) << 10) | ((c & 0x1F) << 8)
    val = raw.view(np.float16).astype(np.float32) * np.float32(4096.0)
    return val.astype(np.float16).view(np.uint16)


def fp6_dequant(stream_i32: np.ndarray, scale: np.ndarray) -> np.ndarray:
    """``dequantize`` of the reference: (n, k*3/16) int32 + (n,) fp16 -> (n, k) fp16.

    Restates ``dequantMatrix_fp6_to_fp16`` (weight_prepacking.cpp:180-217): the exact code value
    times the row's scale with ONE fp16 round-to-nearest multiply.  (The product of two fp16 values
    is exact in fp32, so fp32-multiply-then-round equals ``__hmul``.)
    """
    n = stream_i32.shape[0]
    codes = fp6_unpack_stream(np.ascontiguousarray(stream_i32).view(np.uint8).reshape(n, -1))
    val = fp6_code_to_fp16_bits(codes).view(np.float16).astype(np.float32)
    s = np.asarray(scale).astype(np.float16).astype(np.float32).reshape(n, 1)
    return (val * s).astype(np.float16)


# --------------------------------------------------------------------------------------------
# Reference tensor-core layouts (what the reference kernel consumes)
# --------------------------------------------------------------------------------------------


def _fragment_coords(k: int, n: int):
    """Index grids of the reference's fragment order.

    Weights are cut into chunks of 16 (k) x 64 (n), chunk index ``kb * (n/64) + ch``; lane
    ``4g + t`` of a chunk owns, for sub-tile j (0..3) and half h (0..1), the values v0..v3 at rows
    ``16kb + {2t, 2t+1, 2t+8, 2t+9}`` and column ``64ch + 16j + 8h + g`` - the column operand of an
    m16n8k16 tensor-core tile (test.py:60-79; weight_prepacking.cpp:64-72, 136-150).
    Returns (rows, cols) with shape (k/16, n/64, 32 lanes, 4 j, 2 h, 4 v).
    """
    kb = np.arange(k // 16).reshape(-1, 1, 1, 1, 1, 1)
    ch = np.arange(n // 64).reshape(1, -1, 1, 1, 1, 1)
    lane = np.arange(32).reshape(1, 1, -1, 1, 1, 1)
    j = np.arange(4).reshape(1, 1, 1, -1, 1, 1)
    h = np.arange(2).reshape(1, 1, 1, 1, -1, 1)
    v = np.arange(4).reshape(1, 1, 1, 1, 1, -1)
    g, t = lane // 4, lane % 4
    rows = 16 * kb + 2 * t + (v % 2) + 8 * (v // 2)
    cols = 64 * ch + 16 * j + 8 * h + g
    rows, cols = np.broadcast_arrays(rows, cols)
    return rows, cols


def int4_pack_reference(q: np.ndarray) -> np.ndarray:
    """INT4 codes q[k, n] in 0..15 -> the reference layout, (k/16, 2n) int32.

    Restates the packing half of ``gen_int4_weight`` (test.py:106-114) with ``get_perms``
    (test.py:60-83): four u32 per lane per chunk at word ``(chunk*32 + lane)*4 + j``; nibbles from
    the least significant are v0, v2, v4, v6, v1, v3, v5, v7 with v0..3 = half 0 and v4..7 = half 1.
    """
    k, n = q.shape
    assert k % 16 == 0 and n % 64 == 0
    rows, cols = _fragment_coords(k, n)
    vals = q[rows, cols].astype(np.uint32)                      # (kb, ch, lane, j, h, v)
    vals = vals.reshape(k // 16, n // 64, 32, 4, 8)             # v index = 4h + v
    order = [0, 2, 4, 6, 1, 3, 5, 7]
    word = np.zeros(vals.shape[:-1], dtype=np.uint32)
    for pos, src in enumerate(order):
        word |= vals[..., src] << np.uint32(4 * pos)
    return word.reshape(k // 16, n * 2).view(np.int32)


def int4_unpack_reference(packed: np.ndarray, k: int, n: int) -> np.ndarray:
    """Inverse of :func:`int4_pack_reference`: (k/16, 2n) int32 -> q[k, n] uint8."""
    word = np.ascontiguousarray(packed).view(np.uint32).reshape(k // 16, n // 64, 32, 4)
    order = [0, 2, 4, 6, 1, 3, 5, 7]
    vals = np.zeros(word.shape + (8,), dtype=np.uint8)
    for pos, src in enumerate(order):
        vals[..., src] = (word >> np.uint32(4 * pos)) & 0xF
    rows, cols = _fragment_coords(k, n)
    q = np.zeros((k, n), dtype=np.uint8)
    q[rows, cols] = vals.reshape(rows.shape)
    return q


SCALE_PERM = [2 * i + j for i in range(4) for j in (0, 1, 8, 9, 16, 17, 24, 25)]   # test.py:48-53, 80-83


def permute_scales_reference(s: np.ndarray) -> np.ndarray:
    """Per-column scales (n,) -> the order the reference kernel reads (test.py:48-53, 103-105)."""
    return s.reshape(-1, 32)[:, SCALE_PERM].reshape(-1)


def unpermute_scales_reference(s: np.ndarray) -> np.ndarray:
    inv = np.argsort(np.array(SCALE_PERM))
    return s.reshape(-1, 32)[:, inv].reshape(-1)


def fp6_prepack_reference(stream_i32: np.ndarray) -> np.ndarray:
    """``prepacking`` of the reference: (n, k*3/16) int32 stream -> (k*3/32, 2n) int32 "2+4" layout.

    Restates ``weight_matrix_prepacking`` (weight_prepacking.cpp:123-177): all 2-bit planes
    (k*n/4 bytes; two u32 per lane per chunk at word ``(chunk*32 + lane)*2 + j/2``) followed by all
    4-bit planes (k*n/2 bytes; four u32 per lane per chunk at ``(chunk*32 + lane)*4 + j``).  With
    each code written as the byte ``s eee mm 0 0`` and the four bytes of a (j, h) group laid
    most-significant first as v1, v3, v0, v2, the top two bits of every byte go to the 2-bit word
    at bit offset ``4*(j&1) + 2h`` below the byte's top, and the middle four bits go to the high
    (h=0) or low (h=1) nibble of the same byte of the 4-bit word - the split that
    ``dequant_8fp6`` undoes (fp6_marlin_cuda_kernel.cu:195-237, 575-583).
    """
    n = stream_i32.shape[0]
    codes_nk = fp6_unpack_stream(np.ascontiguousarray(stream_i32).view(np.uint8).reshape(n, -1))
    k = codes_nk.shape[1]
    assert n % 64 == 0 and k % 64 == 0
    code_kn = codes_nk.T                                           # logical [k, n]
    rows, cols = _fragment_coords(k, n)
    c = code_kn[rows, cols].astype(np.uint32)                      # (kb, ch, lane, j, h, v)
    byte_of_v = {1: 3, 3: 2, 0: 1, 2: 0}                           # v -> byte index (0 = least significant)
    w4 = np.zeros(c.shape[:4], dtype=np.uint32)                    # (kb, ch, lane, j)
    w2 = np.zeros(c.shape[:3] + (2,), dtype=np.uint32)             # (kb, ch, lane, j/2)
    for j in range(4):
        for h in range(2):
            for v in range(4):
                code = c[:, :, :, j, h, v]
                by = byte_of_v[v]
                lo4 = code & 0xF
                hi2 = code >> 4
                w4[:, :, :, j] |= lo4 << np.uint32(8 * by + (4 if h == 0 else 0))
                w2[:, :, :, j // 2] |= hi2 << np.uint32(8 * by + 6 - (4 * (j & 1) + 2 * h))
    out = np.concatenate([w2.reshape(-1), w4.reshape(-1)]).view(np.int32)
    return out.reshape(k * 3 // 32, n * 2)


def fp6_unpack_reference(packed: np.ndarray, k: int, n: int) -> np.ndarray:
    """Inverse of :func:`fp6_prepack_reference`: "2+4" layout -> logical codes[k, n] (uint8)."""
    flat = np.ascontiguousarray(packed).view(np.uint32).reshape(-1)
    n2 = k * n // 16
    w2 = flat[:n2].reshape(k // 16, n // 64, 32, 2)
    w4 = flat[n2:].reshape(k // 16, n // 64, 32, 4)
    byte_of_v = {1: 3, 3: 2, 0: 1, 2: 0}
    c = np.zeros((k // 16, n // 64, 32, 4, 2, 4), dtype=np.uint8)
    for j in range(4):
        for h in range(2):
            for v in range(4):
                by = byte_of_v[v]
                lo4 = (w4[:, :, :, j] >> np.uint32(8 * by + (4 if h == 0 else 0))) & 0xF
                hi2 = (w2[:, :, :, j // 2] >> np.uint32(8 * by + 6 - (4 * (j & 1) + 2 * h))) & 0x3
                c[:, :, :, j, h, v] = ((hi2 << 4) | lo4).astype(np.uint8)
    rows, cols = _fragment_coords(k, n)
    codes = np.zeros((k, n), dtype=np.uint8)
    codes[rows, cols] = c
    return codes


# --------------------------------------------------------------------------------------------
# Quantisers (logical level)
# --------------------------------------------------------------------------------------------


def _f16(x):
    return np.asarray(x, dtype=np.float16)


def int4_quantize_per_channel(w: np.ndarray):
    """Reference INT4 rule (test.py:85-98): per-column scale ``max|w| * 2/15`` (fp16 arithmetic),
    ``q = clamp(round(w/s) + 8, 0, 15)``, dequantised weight ``(q-8).half() * s``.
    Returns (q uint8 [k, n], s fp16 (n,), w_deq fp16 [k, n])."""
    w = _f16(w)
    s = np.max(np.abs(w), axis=0, keepdims=True)
    s = (s.astype(np.float32) * np.float32(2.0 / 15.0)).astype(np.float16)   # torch: fp16 tensor times a python scalar
    q = np.rint((w.astype(np.float32) / s.astype(np.float32)).astype(np.float16).astype(np.float32))
    q = np.clip(q.astype(np.int32) + 8, 0, 15)
    deq = ((q - 8).astype(np.float32) * s.astype(np.float32)).astype(np.float16)
    return q.astype(np.uint8), s.reshape(-1), deq


def int4_quantize_group(w: np.ndarray, group_size: int = 128):
    """Group-wise symmetric INT4 along k (this format is not in the reference, whose kernel is
    per-channel only, fp6_marlin_cuda_kernel.cu:447-448): ``s = max|w_group| / 7`` in fp16 (1 for an
    all-zero group), ``q = clamp(round(w/s), -8, 7) + 8``, dequantised weight ``fp16(q-8) * s`` with
    one fp16 multiply - the same form as test.py:98.
    Returns (q uint8 [k, n], s fp16 [k/group, n], w_deq fp16 [k, n])."""
    w = _f16(w)
    k, n = w.shape
    assert k % group_size == 0
    wg = w.reshape(k // group_size, group_size, n).astype(np.float32)
    s = (np.max(np.abs(wg), axis=1) / np.float32(7.0)).astype(np.float16)
    s = np.where(s == 0, np.float16(1.0), s)
    sf = s.astype(np.float32)[:, None, :]
    q = np.rint((wg / sf).astype(np.float16).astype(np.float32)).astype(np.int32)
    q = np.clip(q, -8, 7) + 8
    deq = ((q - 8).astype(np.float32) * sf).astype(np.float16).reshape(k, n)
    return q.reshape(k, n).astype(np.uint8), s, deq


def int4_dequant(q: np.ndarray, s: np.ndarray, group_size: int = -1) -> np.ndarray:
    """``fp16(q - 8) * s`` with one fp16 multiply (test.py:98); s is (n,) or (k/group, n)."""
    k, n = q.shape
    v = q.astype(np.float32) - 8.0
    if group_size <= 0:
        sf = np.asarray(s).astype(np.float16).astype(np.float32).reshape(1, n)
    else:
        sf = np.repeat(np.asarray(s).astype(np.float16).astype(np.float32), group_size, axis=0)
    return (v * sf).astype(np.float16)


def fp6_fake_quantize(w: np.ndarray):
    """The FP6 half of the reference's weight generator (test.py:13-27): per-column scale
    ``max|w| / 28`` in fp16, ``x = w / s``, values with ``|x| < 0.0625`` set to zero, clamp to +-28.
    Returns (x fp16 [k, n], s fp16 (n,))."""
    w = _f16(w)
    s = np.max(np.abs(w), axis=0, keepdims=True)
    s = (s.astype(np.float32) * np.float32(1.0 / 28.0)).astype(np.float16)   # torch: fp16 tensor times a python scalar
    x = (w.astype(np.float32) / s.astype(np.float32)).astype(np.float16)
    x = np.where(np.abs(x) < np.float16(FP6_MIN), np.float16(0), x)
    x = np.clip(x, np.float16(-FP6_MAX), np.float16(FP6_MAX))
    return x, s.reshape(-1)


def fp6_codes_and_dequant(w: np.ndarray):
    """fp16 weights W[k, n] -> (codes uint8 [k, n], s fp16 (n,), w_deq fp16 [k, n]) in the faithful
    orientation: the stream holds row n of the (n, k) matrix, so ``dequantize`` returns W^T."""
    x, s = fp6_fake_quantize(w)
    codes = fp6_encode(x)
    val = fp6_code_to_fp16_bits(codes).view(np.float16).astype(np.float32)
    deq = (val * s.astype(np.float32).reshape(1, -1)).astype(np.float16)
    return codes, s, deq


# --------------------------------------------------------------------------------------------
# The definition of "correct" for the GEMM
# --------------------------------------------------------------------------------------------


def gemm_reference(a: np.ndarray, w_deq: np.ndarray) -> np.ndarray:
    """``C = A.float() @ W_deq.float()`` accumulated in fp32 (the check the reference's tests make
    with an fp16 matmul, test.py:167, made stricter)."""
    return a.astype(np.float32) @ w_deq.astype(np.float32)


def rel_frobenius(c: np.ndarray, c_ref: np.ndarray) -> float:
    c = np.asarray(c, dtype=np.float64)
    c_ref = np.asarray(c_ref, dtype=np.float64)
    den = float(np.linalg.norm(c_ref))
    return float(np.linalg.norm(c - c_ref)) / (den if den > 0 else 1.0)

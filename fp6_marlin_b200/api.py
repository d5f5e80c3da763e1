"""Host-side mirror of the reference's ``fp6_marlin`` Python module (fp6_marlin/__init__.py:8-40):
``prepacking``, ``quantize``, ``dequantize`` and ``mul`` with the same names, argument order,
defaults, shapes, dtypes and error behaviour, implemented over the C ABI of libfp6m.so.

Differences from the reference, all additive:
  * shape violations raise ``ValueError`` instead of aborting the interpreter through ``assert``
    (pybind.cpp:22-24, 50);
  * ``mul`` takes two keyword-only arguments: ``group_size`` (128 for INT4 group scales; -1 for the
    reference's per-channel scales) and ``layout`` ("reference" for tensors packed the reference's
    way, "b200" for the Blackwell tiling produced by :func:`fp6_marlin_b200.pack_b200`).
PyTorch is used for memory, streams and device management only.
"""
from __future__ import annotations

import weakref

import torch

from . import _lib
from ._lib import lib


def _ptr(t: torch.Tensor) -> int:
    return t.data_ptr()


# ----------------------------------------------------------------------------------------------
# quantize / prepacking / dequantize (host, weight preparation)
# ----------------------------------------------------------------------------------------------


def quantize(fp16_tensor: torch.Tensor) -> torch.Tensor:
    """Cast fake-quantised fp16 weights to FP6 E3M2 (truncating) and pack 4 codes into 3 bytes.

    Same contract as ``fp6_marlin.quantize`` (fp6_marlin/__init__.py:18-26, pybind.cpp:42-59):
    input (a, b) fp16 on the CPU with a, b multiples of 256 and every value in {0} U [0.0625, 28] in
    magnitude; output (b, a*3/16) int32.  The row-major memory of the input is packed as it lies
    (the reference's transpose is a view only), so pass ``W.t().contiguous().view(k, n)`` to get the
    (n, k)-major stream of a logical ``W[k, n]``.
    """
    if fp16_tensor.dtype != torch.float16:
        raise ValueError("Input tensor should be of type float16.")
    if fp16_tensor.dim() != 2 or fp16_tensor.shape[0] % 256 or fp16_tensor.shape[1] % 256:
        raise ValueError("quantize: expected a 2-D tensor whose dimensions are multiples of 256")
    a, b = fp16_tensor.shape
    src = fp16_tensor.detach().cpu().contiguous()
    out = torch.empty((b, a * 3 // 16), dtype=torch.int32)
    rc = lib.fp6m_quantize_fp6(_ptr(src), _ptr(out), b, a)
    if rc == _lib.ERR_VALUE_RANGE:
        raise ValueError("Input value out of range for FP6.")
    if rc:
        raise RuntimeError(f"fp6m_quantize_fp6 failed with code {rc}")
    return out


def prepacking(fp6_tensor: torch.Tensor) -> torch.Tensor:
    """FP6 stream (n, k*3/16) int32 -> the reference's "2+4" tensor-core layout (k*3/32, 2n) int32,
    byte-identical to ``fp6_marlin.prepacking`` (fp6_marlin/__init__.py:8-16, pybind.cpp:18-31)."""
    if fp6_tensor.dtype != torch.int32 or fp6_tensor.dim() != 2 or fp6_tensor.shape[1] % 3:
        raise ValueError("prepacking: expected an int32 tensor of shape (n, k*3/16)")
    n = fp6_tensor.shape[0]
    k = fp6_tensor.shape[1] * 16 // 3
    if n % 256 or k % 256:
        raise ValueError("prepacking: n and k must be multiples of 256")
    src = fp6_tensor.detach().cpu().contiguous()
    out = torch.empty((k * 3 // 32, n * 2), dtype=torch.int32)
    rc = lib.fp6m_prepack_fp6(_ptr(src), _ptr(out), n, k)
    if rc:
        raise RuntimeError(f"fp6m_prepack_fp6 failed with code {rc}")
    return out


def dequantize(fp6_tensor: torch.Tensor, fp16_scales: torch.Tensor) -> torch.Tensor:
    """FP6 stream (n, k*3/16) int32 + per-row fp16 scales (n,) -> (n, k) fp16, bit-identical to
    ``fp6_marlin.dequantize`` (fp6_marlin/__init__.py:28-37, pybind.cpp:70-87)."""
    if fp6_tensor.dtype != torch.int32 or fp6_tensor.dim() != 2 or fp6_tensor.shape[1] % 3:
        raise ValueError("dequantize: expected an int32 tensor of shape (n, k*3/16)")
    n = fp6_tensor.shape[0]
    k = fp6_tensor.shape[1] * 16 // 3
    if fp16_scales.dtype != torch.float16 or fp16_scales.numel() != n:
        raise ValueError("dequantize: scales must be float16 with one value per row")
    src = fp6_tensor.detach().cpu().contiguous()
    sc = fp16_scales.detach().cpu().contiguous()
    out = torch.empty((n, k), dtype=torch.float16)
    rc = lib.fp6m_dequant_fp6(_ptr(src), _ptr(sc), _ptr(out), n, k)
    if rc:
        raise RuntimeError(f"fp6m_dequant_fp6 failed with code {rc}")
    return out.to(fp16_scales.device)


# ----------------------------------------------------------------------------------------------
# b200 layout helpers
# ----------------------------------------------------------------------------------------------


def b200_sizes(k: int, n: int, quant_cols: int = -1, group_size: int = -1):
    """(int32 words of the packed weight buffer, number of fp16 scales) of the b200 layout."""
    nbytes = lib.fp6m_b200_weight_bytes(k, n, quant_cols)
    nscales = lib.fp6m_b200_scale_count(k, n, quant_cols, group_size)
    if nbytes < 0 or nscales < 0:
        raise ValueError("b200_sizes: bad shape")
    return nbytes // 4, nscales


def pack_b200(q4, c6, s4, s6, k: int, n: int, quant_cols: int = -1, group_size: int = -1):
    """Logical codes -> (B int32 flat, s fp16 flat) in the b200 layout (CPU tensors).

    q4: (k, n - qc) uint8 INT4 codes 0..15 (value q - 8); c6: (k, qc) uint8 FP6 codes;
    s4: (k/128, n - qc) or (n - qc,) fp16; s6: (qc,) fp16.  Either region may be absent (None).
    """
    qc = max(quant_cols, 0)
    words, nscales = b200_sizes(k, n, quant_cols, group_size)
    B = torch.empty(words, dtype=torch.int32)
    s = torch.empty(nscales, dtype=torch.float16)

    def prep(t, dtype, numel):
        if numel == 0:
            return None, 0
        if t is None:
            raise ValueError("pack_b200: a region with columns needs its codes and scales")
        t = t.detach().cpu().contiguous()
        if t.dtype != dtype or t.numel() != numel:
            raise ValueError(f"pack_b200: expected {numel} elements of {dtype}, got {t.numel()} of {t.dtype}")
        return t, _ptr(t)

    groups = (k + 127) // 128 if group_size > 0 else 1
    q4_t, q4_p = prep(q4, torch.uint8, k * (n - qc))
    c6_t, c6_p = prep(c6, torch.uint8, k * qc)
    s4_t, s4_p = prep(s4, torch.float16, groups * (n - qc))
    s6_t, s6_p = prep(s6, torch.float16, qc)
    rc = lib.fp6m_pack_b200(q4_p, c6_p, s4_p, s6_p, k, n, quant_cols, group_size, _ptr(B), _ptr(s))
    if rc:
        raise RuntimeError(f"fp6m_pack_b200 failed with code {rc}")
    return B, s


def pack_b200_gpu(q4, c6, s4, s6, k: int, n: int, quant_cols: int = -1, group_size: int = -1):
    """:func:`pack_b200` on the GPU: CUDA tensors in, (B, s) on the same device out, same bytes.
    Asynchronous on the current stream; padding bytes of the buffers are zero."""
    qc = max(quant_cols, 0)
    device = next(t.device for t in (q4, c6, s4, s6) if t is not None)
    if device.type != "cuda":
        raise ValueError("pack_b200_gpu: the inputs must be CUDA tensors")
    words, nscales = b200_sizes(k, n, quant_cols, group_size)
    B = torch.zeros(words, dtype=torch.int32, device=device)
    s = torch.zeros(nscales, dtype=torch.float16, device=device)

    def prep(t, dtype, numel):
        if numel == 0:
            return None, 0
        if t is None:
            raise ValueError("pack_b200_gpu: a region with columns needs its codes and scales")
        t = t.detach().to(device).contiguous()
        if t.dtype != dtype or t.numel() != numel:
            raise ValueError(f"pack_b200_gpu: expected {numel} elements of {dtype}, got {t.numel()} of {t.dtype}")
        return t, _ptr(t)

    groups = (k + 127) // 128 if group_size > 0 else 1
    q4_t, q4_p = prep(q4, torch.uint8, k * (n - qc))
    c6_t, c6_p = prep(c6, torch.uint8, k * qc)
    s4_t, s4_p = prep(s4, torch.float16, groups * (n - qc))
    s6_t, s6_p = prep(s6, torch.float16, qc)
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream(device).cuda_stream
        rc = lib.fp6m_pack_b200_device(q4_p, c6_p, s4_p, s6_p, k, n, quant_cols, group_size, _ptr(B), _ptr(s),
                                       device.index if device.index is not None else torch.cuda.current_device(), stream)
    if rc:
        raise RuntimeError(f"fp6m_pack_b200_device failed with code {rc}: {_lib.last_cuda_error()}")
    return B, s


def encode_fp6_gpu(x: torch.Tensor) -> torch.Tensor:
    """fp16 CUDA tensor of values in the FP6 range -> codes ``s eee mm`` (uint8) on the same device, the
    truncating cast of the reference (weight_quant.cpp:27-91).  Raises ``ValueError`` for out-of-range
    input like the host function (this check synchronises)."""
    if x.dtype != torch.float16:
        raise ValueError("Input tensor should be of type float16.")
    if x.device.type != "cuda":
        raise ValueError("encode_fp6_gpu: the input must be a CUDA tensor")
    src = x.detach().contiguous()
    codes = torch.empty(src.shape, dtype=torch.uint8, device=src.device)
    flag = torch.zeros(1, dtype=torch.int32, device=src.device)
    with torch.cuda.device(src.device):
        rc = lib.fp6m_encode_fp6_device(_ptr(src), _ptr(codes), src.numel(), src.device.index,
                                        torch.cuda.current_stream(src.device).cuda_stream, _ptr(flag))
    if rc:
        raise RuntimeError(f"fp6m_encode_fp6_device failed with code {rc}")
    if int(flag.item()) == _lib.ERR_VALUE_RANGE:
        raise ValueError("Input value out of range for FP6.")
    return codes


def unpack_b200(B: torch.Tensor, s: torch.Tensor, k: int, n: int, quant_cols: int = -1, group_size: int = -1):
    """Inverse of :func:`pack_b200`: returns (q4, c6, s4, s6) as CPU tensors."""
    qc = max(quant_cols, 0)
    groups = (k + 127) // 128 if group_size > 0 else 1
    B = B.detach().cpu().contiguous()
    s = s.detach().cpu().contiguous()
    q4 = torch.zeros((k, n - qc), dtype=torch.uint8)
    c6 = torch.zeros((k, qc), dtype=torch.uint8)
    s4 = torch.zeros((groups, n - qc), dtype=torch.float16)
    s6 = torch.zeros((qc,), dtype=torch.float16)
    rc = lib.fp6m_unpack_b200(_ptr(B), _ptr(s), k, n, quant_cols, group_size,
                              _ptr(q4) if q4.numel() else 0, _ptr(c6) if c6.numel() else 0,
                              _ptr(s4) if s4.numel() else 0, _ptr(s6) if s6.numel() else 0)
    if rc:
        raise RuntimeError(f"fp6m_unpack_b200 failed with code {rc}")
    return q4, c6, s4, s6


def repack_from_reference(B_ref: torch.Tensor, s_ref: torch.Tensor, k: int, n: int, quant_cols: int = -1):
    """Tensors packed the reference's way (``gen_mixed_weight``, test.py:123-152: INT4 words, then
    FP6 "2+4" words; permuted per-channel scales) -> (B, s) in the b200 layout on the same device."""
    qc = max(quant_cols, 0)
    dev = B_ref.device
    src = B_ref.detach().cpu().contiguous()
    sc = s_ref.detach().cpu().contiguous()
    if sc.dtype != torch.float16 or sc.numel() != n:
        raise ValueError("repack_from_reference: s must hold one float16 per column")
    if src.numel() * src.element_size() != k * (n - qc) // 2 + k * qc * 3 // 4:
        raise ValueError("repack_from_reference: B has the wrong size for this shape")
    words, nscales = b200_sizes(k, n, quant_cols, -1)
    B = torch.empty(words, dtype=torch.int32)
    s = torch.empty(nscales, dtype=torch.float16)
    rc = lib.fp6m_repack_from_reference(_ptr(src), _ptr(sc), k, n, quant_cols, _ptr(B), _ptr(s))
    if rc == _lib.ERR_PROB_SHAPE:
        raise ValueError("repack_from_reference: k must be a multiple of 16 and both regions multiples of 64 columns")
    if rc:
        raise RuntimeError(f"fp6m_repack_from_reference failed with code {rc}")
    return B.to(dev), s.to(dev)


def schedule(k: int, n: int, quant_cols: int = -1, group_size: int = -1, ctas: int = 148):
    """Block boundaries of the stripe schedule (list of ctas+1 ints) and the number of blocks."""
    import ctypes
    buf = (ctypes.c_int * (ctas + 1))()
    total = lib.fp6m_schedule(k, n, quant_cols, group_size, ctas, buf)
    if total < 0:
        raise ValueError("schedule: bad arguments")
    return list(buf), total


def launch_plan(m: int, n: int, k: int, quant_cols: int = -1, sms: int = 148):
    """How `mul` cuts the shape into kernel launches on a device with `sms` multiprocessors: (number of
    launches, True if the kernel for more than 128 rows runs)."""
    import ctypes
    many = ctypes.c_int(0)
    launches = lib.fp6m_mul_launches(m, n, k, quant_cols, sms, ctypes.byref(many))
    return launches, bool(many.value)


# ----------------------------------------------------------------------------------------------
# mul
# ----------------------------------------------------------------------------------------------

_scratch: dict[tuple[int, int], torch.Tensor] = {}
_status: dict[int, torch.Tensor] = {}
_sm_count: dict[int, int] = {}
_prepared: dict[int, tuple] = {}


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_scratch_need: dict[tuple, int] = {}


def _stream_handle(idx: int, device: torch.device) -> int:
    """The cudaStream_t of the current torch stream of `device`."""
    if _raw_stream is not None:
        return _raw_stream(idx)
    return torch.cuda.current_stream(device).cuda_stream


def _device_buffers(device: torch.device, shape=None, stream=None):
    """(device index, split-K scratch, status word) for a GEMM on the CURRENT stream of `device`
    (`stream`: its handle, if the caller has it already).

    The scratch holds the launch epoch and the tagged split-K slots of the kernels, so two GEMMs that
    can overlap on the GPU must not share one: there is one buffer per (device, stream), created (and
    zeroed, in stream order) the first time a stream is used and grown when a shape needs more.
    `shape` = (M, N, K, quant_cols) sizes it for that GEMM; None sizes it for any GEMM of up to 16 rows.
    The reference is re-entrant per stream in the same way: each concurrent call brings its own
    workspace (fp6_marlin_cuda_kernel.cu:90-93)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=device)
        _sm_count[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    need_key = (idx, shape)
    nbytes = _scratch_need.get(need_key)
    if nbytes is None:
        if shape is None:
            nbytes = lib.fp6m_mul_scratch_bytes(16, 1 << 20, 1 << 14, 0, _sm_count[idx])
        else:
            nbytes = lib.fp6m_mul_scratch_bytes(shape[0], shape[1], shape[2], shape[3], _sm_count[idx])
        if len(_scratch_need) > 4096:
            _scratch_need.clear()
        _scratch_need[need_key] = nbytes
    key = (idx, _stream_handle(idx, device) if stream is None else stream)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        # zero once: the kernels keep the epoch and the tagged slots in it between calls
        with torch.cuda.device(device):
            buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return idx, buf, _status[idx]


def set_launch_overlap(enable: bool) -> bool:
    """Process-wide switch for programmatic dependent launch of the GEMM kernels (off by default);
    returns the previous setting.  When on, a GEMM may set itself up and prefetch its weights while the
    kernel before it in the stream is finishing; A, C and the scratch are only touched after that kernel
    has completed.  Only turn it on when the kernel preceding a GEMM in its stream does not write that
    GEMM's weights or scales."""
    return bool(lib.fp6m_set_launch_overlap(1 if enable else 0))


def set_ordered_sums(enable: bool) -> bool:
    """Process-wide switch (off by default); returns the previous setting.  When on, the GEMM for up to 16
    rows adds the products of a 128-row block in one fixed order, so two runs on the same inputs agree bit
    for bit; when off, the two 64-row halves of a block may be added in either order (faster)."""
    return bool(lib.fp6m_set_ordered_sums(1 if enable else 0))


def device_status(device=None) -> int:
    """Reads (and clears) the device status word: 0, or FP6M_ERR_TIMEOUT (8) if a bounded wait
    inside a kernel ran out since the last call.  Synchronises the device."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status:
        return 0
    status = _status[idx]
    value = int(status.item())
    if value:
        status.zero_()
    return value


def _prepared_from_reference(B, s, k, n, quant_cols):
    """Reference-layout tensors are re-tiled once and remembered for as long as `B` lives and is
    not modified in place."""
    key = id(B)
    hit = _prepared.get(key)
    if hit is not None:
        ref, ver, s_ref, s_ver, shape, packed = hit
        if ref() is B and ver == B._version and s_ref() is s and s_ver == s._version and shape == (k, n, quant_cols):
            return packed
    packed = repack_from_reference(B, s, k, n, quant_cols)
    _prepared[key] = (weakref.ref(B, lambda _r, key=key: _prepared.pop(key, None)), B._version,
                      weakref.ref(s), s._version, (k, n, quant_cols), packed)
    return packed


def mul(A, B, C, s, workspace, quant_cols=-1, thread_k=-1, thread_n=-1, sms=-1, max_par=16, *,
        group_size=-1, layout="reference"):
    """``C[M, N] = A[M, K] @ dequant(B, s)``: FP16 activations times mixed INT4 / FP6 weights.

    Same contract as ``fp6_marlin.mul`` (fp6_marlin/__init__.py:39-40, fp6_marlin_cuda.cpp:47-92):
    A (M, K) fp16, B packed int32, C (M, N) fp16 pre-allocated and overwritten in place, s fp16
    scales, workspace with at least ``N/128*max_par`` zero-filled 4-byte elements (left zero), all
    on one CUDA device; runs asynchronously on the current stream of A's device and returns None.
    Calls on different streams of one device may overlap: each stream has its own split-K scratch.
    The last ``quant_cols`` columns of B are FP6 (``-1``: none; ``N``: all), and C keeps B's column
    order.  Raises ``RuntimeError`` for the cases the reference raises for: workspace too small,
    ``N % thread_n`` or ``K % thread_k`` non-zero, no kernel for the tile shape.
    """
    if not A.is_cuda:
        raise RuntimeError("fp6_marlin_b200.mul needs CUDA tensors: there is no CPU implementation")
    M, K = A.shape[0], A.shape[1]
    N = C.shape[1]
    if workspace.numel() < N // 128 * max_par:
        raise RuntimeError(f"workspace must be of size at least {N // 128 * max_par}.")
    if A.dtype != torch.float16 or C.dtype != torch.float16 or s.dtype != torch.float16:
        raise RuntimeError("mul: A, C and s must be float16")
    if not (A.is_contiguous() and C.is_contiguous() and B.is_contiguous() and s.is_contiguous()):
        raise RuntimeError("mul: tensors must be contiguous")
    if C.shape[0] != M:
        raise RuntimeError("mul: C must have as many rows as A")

    if layout == "reference":
        # the reference validates tile shapes before it touches B: keep its error order
        tk, tn = (thread_k, thread_n)
        if tk == -1 or tn == -1:
            tk, tn = (128, 128) if M <= 16 else (64, 256)
        if tk > 0 and tn > 0 and (N % tn or K % tk):
            raise RuntimeError(f"Problem (m={M}, n={N}, k={K}) not compatible with thread_k={thread_k}, thread_n={thread_n}.")
        if not ((tk == 128 and tn == 128 and M <= 16) or (tk == 64 and tn == 256)):
            raise RuntimeError(f"No kernel implementation for thread_k={thread_k}, thread_n={thread_n}.")
        if M == 0 or N == 0 or K == 0:
            return
        if group_size > 0:
            raise RuntimeError("mul: the reference layout has per-channel scales only (group_size=-1)")
        B, s = _prepared_from_reference(B, s, K, N, quant_cols)
    elif layout != "b200":
        raise RuntimeError(f"mul: unknown layout {layout!r}")

    device = A.device
    stream = _stream_handle(device.index if device.index is not None else torch.cuda.current_device(), device)
    dev_index, scratch, status = _device_buffers(device, (M, N, K, quant_cols), stream)
    rc = lib.fp6m_mul(_ptr(A), _ptr(B), _ptr(C), _ptr(s), M, N, K,
                      _ptr(workspace), workspace.numel() * workspace.element_size(),
                      _ptr(scratch), scratch.numel(), dev_index, stream,
                      thread_k, thread_n, sms, max_par, quant_cols, group_size, _lib.LAYOUT_B200, _ptr(status))
    if rc == _lib.OK:
        return
    if rc == _lib.ERR_PROB_SHAPE:
        raise RuntimeError(f"Problem (m={M}, n={N}, k={K}) not compatible with thread_k={thread_k}, thread_n={thread_n}.")
    if rc == _lib.ERR_KERN_SHAPE:
        raise RuntimeError(f"No kernel implementation for thread_k={thread_k}, thread_n={thread_n}.")
    if rc == _lib.ERR_WORKSPACE:
        raise RuntimeError(f"workspace must be of size at least {N // 128 * max_par}.")
    if rc == _lib.ERR_CUDA:
        raise RuntimeError(f"fp6m_mul: CUDA error: {_lib.last_cuda_error()}")
    raise RuntimeError(f"fp6m_mul failed with code {rc}")


def mul_fused(A, B, C, s, workspace, quant_cols=-1, *, epilogue="none", residual=None, sms=-1, max_par=16,
              group_size=-1):
    """``mul`` (b200 layout only) with the step that follows the GEMM in a transformer block fused into its
    epilogue, applied to the fp32 sums before the single rounding to fp16:

    ``epilogue="silu_mul"``  gate / up projection: B holds the two projections interleaved - columns 2j and
                             2j+1 of the INT4 region, and of the FP6 region, are gate_j and up_j (see
                             :func:`fp6_marlin_b200.make_gate_up_weight`) - and C, of shape (M, N/2),
                             receives ``silu(gate_j) * up_j``: INT4 pairs first, then FP6 pairs.
    ``epilogue="residual"``  ``C = A @ W + residual`` with ``residual`` an (M, N) fp16 tensor (it may be C).

    The reference only scales and stores (write_result, fp6_marlin_cuda_kernel.cu:698-749); the layers on
    either side of its GEMM are the ones its benchmark lists (bench.py:53-86).
    """
    code = {"none": _lib.EPILOGUE_NONE, "silu_mul": _lib.EPILOGUE_SILU_MUL, "residual": _lib.EPILOGUE_RESIDUAL}.get(epilogue)
    if code is None:
        raise ValueError(f"mul_fused: unknown epilogue {epilogue!r}")
    if not A.is_cuda:
        raise RuntimeError("fp6_marlin_b200.mul_fused needs CUDA tensors: there is no CPU implementation")
    M, K = A.shape
    N = C.shape[1] * 2 if code == _lib.EPILOGUE_SILU_MUL else C.shape[1]
    if workspace.numel() < N // 128 * max_par:
        raise RuntimeError(f"workspace must be of size at least {N // 128 * max_par}.")
    if A.dtype != torch.float16 or C.dtype != torch.float16 or s.dtype != torch.float16:
        raise RuntimeError("mul_fused: A, C and s must be float16")
    if not (A.is_contiguous() and C.is_contiguous() and B.is_contiguous() and s.is_contiguous()):
        raise RuntimeError("mul_fused: tensors must be contiguous")
    if C.shape[0] != M:
        raise RuntimeError("mul_fused: C must have as many rows as A")
    res_ptr = 0
    if code == _lib.EPILOGUE_RESIDUAL:
        if residual is None or residual.dtype != torch.float16 or tuple(residual.shape) != (M, N) or not residual.is_contiguous():
            raise RuntimeError("mul_fused: residual must be a contiguous float16 tensor of C's shape")
        res_ptr = _ptr(residual)
    if M == 0 or N == 0 or K == 0:
        return
    device = A.device
    stream = _stream_handle(device.index if device.index is not None else torch.cuda.current_device(), device)
    dev_index, scratch, status = _device_buffers(device, (M, N, K, quant_cols), stream)
    rc = lib.fp6m_mul_fused(_ptr(A), _ptr(B), _ptr(C), _ptr(s), M, N, K,
                            _ptr(workspace), workspace.numel() * workspace.element_size(),
                            _ptr(scratch), scratch.numel(), dev_index, stream,
                            -1, -1, sms, max_par, quant_cols, group_size, _lib.LAYOUT_B200, _ptr(status), code, res_ptr)
    if rc == _lib.ERR_CUDA:
        raise RuntimeError(f"fp6m_mul_fused: CUDA error: {_lib.last_cuda_error()}")
    if rc:
        raise RuntimeError(f"fp6m_mul_fused failed with code {rc}")


def dump_operands(B: torch.Tensor, s: torch.Tensor, k: int, n: int, quant_cols: int = -1, group_size: int = -1):
    """The fp16 matrix W_deq[k, n] that the GEMM kernels feed the tensor cores (b200 layout in)."""
    W = torch.zeros((k, n), dtype=torch.float16, device=B.device)
    dev_index = B.device.index if B.device.index is not None else torch.cuda.current_device()
    stream = torch.cuda.current_stream(B.device).cuda_stream
    rc = lib.fp6m_dump_operands(_ptr(B), _ptr(s), _ptr(W), n, k, quant_cols, group_size, dev_index, stream)
    if rc:
        raise RuntimeError(f"fp6m_dump_operands failed with code {rc}: {_lib.last_cuda_error()}")
    return W

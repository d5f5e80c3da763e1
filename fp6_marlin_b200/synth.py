"""Seeded synthetic layers with the shapes and value distributions the benchmark configurations
name: activations ~ N(0, 1), weights ~ N(0, 0.02) with ``quant_cols`` randomly chosen output
columns scaled x8 as outliers; the ``quant_cols`` columns of largest abs-max become FP6 (moved to
the end, order otherwise kept), the rest INT4.  The reference benchmarks with random bits and
never checks results (bench.py:25-33); these layers are checkable stand-ins of the same shapes.
"""
from __future__ import annotations

import torch

from .quant import W46Weight, make_w46_weight, select_outlier_columns

# (K, N) of the layer sets the configurations name
LLAMA2_7B = {"qkv": (4096, 12288), "o_proj": (4096, 4096), "gate_up": (4096, 22016), "down": (11008, 4096)}
LLAMA2_70B = {"qkv": (8192, 10240), "o_proj": (8192, 8192), "gate_up": (8192, 57344), "down": (28672, 8192)}


def make_weight_fp16(k: int, n: int, quant_cols: int, seed: int = 0, device=None) -> torch.Tensor:
    """fp16 W[k, n] with the outlier columns already moved to the end.  With a CUDA ``device`` the values
    are drawn and kept there (another stream of random numbers than on the CPU, equally seeded)."""
    dev = torch.device("cpu") if device is None else torch.device(device)
    gen = torch.Generator(device=dev).manual_seed(seed)
    w = (torch.randn((k, n), generator=gen, dtype=torch.float32, device=dev) * 0.02)
    qc = max(quant_cols, 0)
    if qc:
        cols = torch.randperm(n, generator=gen, device=dev)[:qc]
        w[:, cols] *= 8.0
    w = w.half()
    if qc:
        w = w[:, select_outlier_columns(w, qc)].contiguous()
    return w


def make_activations(m: int, k: int, seed: int = 0) -> torch.Tensor:
    gen = torch.Generator(device="cpu").manual_seed(1000003 + seed)
    return torch.randn((m, k), generator=gen, dtype=torch.float32).half()


def make_layer(k: int, n: int, quant_cols: int = 256, group_size: int = 128, seed: int = 0,
               keep_dequantized: bool = True, quant_device=None) -> W46Weight:
    """One quantised and packed layer (CPU tensors) in the b200 layout."""
    return make_w46_weight(make_weight_fp16(k, n, quant_cols, seed), quant_cols, group_size, keep_dequantized,
                           quant_device)


def algorithmic_bytes(m: int, k: int, n: int, quant_cols: int, group_size: int) -> int:
    """Bytes a perfect kernel must move: A, packed INT4, packed FP6, scales, C
    (the same form as the reference's bench.py:46-50)."""
    qc = max(quant_cols, 0)
    groups = k // 128 if group_size > 0 else 1
    return 2 * m * k + k * (n - qc) // 2 + k * qc * 3 // 4 + 2 * groups * (n - qc) + 2 * qc + 2 * m * n


def flops(m: int, k: int, n: int) -> int:
    return 2 * m * n * k

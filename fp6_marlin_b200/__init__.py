"""B200-native W(4&6)A16 GEMM: FP16 activations x mixed INT4 / FP6-E3M2 weights.

The four callables of the reference's ``fp6_marlin`` module (``prepacking``, ``quantize``,
``dequantize``, ``mul``) with the same signatures, plus helpers for the Blackwell weight layout.
All compute runs in libfp6m.so (hand-written sm_100a CUDA + host C++) through a C ABI; importing
this package fails if that library has not been built - there is no fallback path.
"""
from .api import (b200_sizes, dequantize, device_status, dump_operands, encode_fp6_gpu, launch_plan, mul, mul_fused, pack_b200, pack_b200_gpu,
                  prepacking,
                  quantize, repack_from_reference, schedule, set_launch_overlap, set_ordered_sums, unpack_b200)
from .linear import W46Linear
from .quant import (W46Weight, decode_fp6, encode_fp6, fake_quantize_fp6, make_gate_up_weight, make_w46_weight,
                    quantize_fp6, quantize_int4, select_outlier_columns)

__all__ = [
    "prepacking", "quantize", "dequantize", "mul", "mul_fused", "make_gate_up_weight",
    "b200_sizes", "pack_b200", "pack_b200_gpu", "encode_fp6_gpu", "unpack_b200", "repack_from_reference", "schedule", "launch_plan", "dump_operands",
    "device_status", "set_launch_overlap", "set_ordered_sums", "W46Linear", "W46Weight", "make_w46_weight", "quantize_int4", "quantize_fp6", "encode_fp6",
    "decode_fp6", "fake_quantize_fp6", "select_outlier_columns",
]

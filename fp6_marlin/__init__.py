"""Drop-in name: ``import fp6_marlin`` resolves to the B200-native implementation, exposing the
reference module's four callables (fp6_marlin/__init__.py:8-40 of the reference project)."""
from fp6_marlin_b200 import dequantize, mul, prepacking, quantize  # noqa: F401

__all__ = ["prepacking", "quantize", "dequantize", "mul"]

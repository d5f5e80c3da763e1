"""Drop-in name of the reference's host extension module: ``quantization_cpu``, ``prepacking_cpu`` and
``dequantization_cpu`` with the signatures of the reference binding (fp6_marlin/pybind.cpp:89-94), served by
the host functions of the B200-native library."""
from fp6_marlin_b200.api import dequantize as dequantization_cpu  # noqa: F401
from fp6_marlin_b200.api import prepacking as prepacking_cpu  # noqa: F401
from fp6_marlin_b200.api import quantize as quantization_cpu  # noqa: F401

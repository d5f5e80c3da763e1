"""Drop-in name of the reference's CUDA extension module: ``fp6_marlin_cuda.mul`` with the positional
signature of the reference binding (fp6_marlin/fp6_marlin_cuda.cpp:47-58, 125-127; max_par defaults to 8
there, to 16 in its Python wrapper), served by the B200-native implementation."""
from fp6_marlin_b200.api import mul as _mul


def mul(A, B, C, s, workspace, quant_cols=-1, thread_k=-1, thread_n=-1, sms=-1, max_par=8):
    return _mul(A, B, C, s, workspace, quant_cols, thread_k, thread_n, sms, max_par)

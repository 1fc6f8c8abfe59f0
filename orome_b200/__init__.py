"""orome_b200 -- B200 (sm_100a) implementation of Orome's quantized dequant-matvec path.

The product is ``liborome_cuda.so`` (C ABI declared in ``include/orome_cuda.h``);
this package is a thin ctypes binding over it plus synthetic-tensor generators.
There is no CPU or PyTorch fallback: importing :mod:`orome_b200.format` without the
built library raises, and every compute call goes to the CUDA kernels.
"""
from .synth import Q4_K, Q5_K, Q6_K, Q8_0, F16, BF16, F32  # noqa: F401

__all__ = ["Q4_K", "Q5_K", "Q6_K", "Q8_0", "F16", "BF16", "F32"]

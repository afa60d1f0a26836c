"""recpulse_b200: Blackwell-native dense matmul (forward + autograd backward) for RecPulse.

The product is ``librecpulse_b200.so`` (C ABI in ``include/recpulse_b200.h``).
This package holds its sources (``csrc/``), the build step, a ctypes binding and a
small mirror of the RecPulse tensor interface for the matmul path.
"""
from . import _lib
from ._lib import BF16, F16, F32, F64, RpbGemm, load
from .tensor import Tensor, from_numpy

__all__ = ["Tensor", "from_numpy", "load", "RpbGemm", "F32", "F64", "F16", "BF16", "_lib"]

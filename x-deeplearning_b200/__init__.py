"""B200-native backend for Blaze's CTR-inference hot path.

The product is two shared libraries built from csrc/ and host/:
  lib/libxdlb200.so    C-ABI CUDA kernels (include/xdlb200.h)
  lib/libblaze_b200.so C++ host runtime mirroring Blaze's Operator / Predictor API
This Python package only binds them with ctypes for tests and benchmarks; it
holds no compute of its own and fails loudly when the libraries are missing.
"""
from . import capi  # noqa: F401
from .capi import lib, build_native  # noqa: F401

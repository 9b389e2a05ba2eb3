"""canopy-foundry_b200: sm_100a implementation of Canopy-Foundry's FP8 quantize-and-GEMM path.

The product is libcanopy_fp8.so (C ABI in include/canopy_fp8.h, sources in csrc/). This package is
the Python-side mirror of the reference's operator interface used by tests and the benchmark:
`ops` exposes the same operator names as include/ida_native/kernels.hpp on torch CUDA tensors.

The directory name contains a hyphen, so import it with importlib:
    cfb = importlib.import_module("canopy-foundry_b200")
"""
from . import _capi
from . import ops
from . import parallel
from .ops import *  # noqa: F401,F403

__all__ = ["_capi", "ops", "parallel"] + ops.__all__

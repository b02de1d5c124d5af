"""miori_b200: B200 (sm_100a) kernels for Miori's quantized-matmul path.

The product is libmiori_b200.so (C ABI in include/miori_b200.h) plus the C++ operator shim
under shim/ that mirrors the reference's src/ops.h.  This package is the thin Python
binding used by the tests and the benchmark.
"""
from . import _lib
from ._lib import GEMV_EXACT, LAUNCH_PDL, OUT_BF16, OUT_F32, MioriError, lib
from .ops import (dequant4_cache, dequant4_rowmajor, dequant8_rowmajor, gemm_bf16_cache, gemv4,
                  gemv8)

__all__ = [
    "lib", "MioriError", "OUT_F32", "OUT_BF16", "LAUNCH_PDL", "GEMV_EXACT", "gemv4", "gemv8",
    "dequant4_rowmajor", "dequant8_rowmajor", "dequant4_cache", "gemm_bf16_cache",
]

"""miori_b200: B200 (sm_100a) kernels for Miori's quantized-matmul path.

The product is libmiori_b200.so (C ABI in include/miori_b200.h) plus the C++ operator shim
under shim/ that mirrors the reference's src/ops.h.  This package is the thin Python
binding used by the tests and the benchmark.

The binding is loaded on first use of any operator or of `lib`; if libmiori_b200.so is
missing or lacks a declared symbol that access raises -- there is no CPU fallback.
`miori_b200.build` (the nvcc driver) imports without the library so that it can create it.
"""
import importlib

_OPS = ("gemv4", "gemv8", "dequant4_rowmajor", "dequant8_rowmajor", "dequant4_cache",
        "cache_to_rowmajor", "gemm_bf16_cache", "gemv_bf16_cache", "gemm_workspace", "gemm_bf16_strided", "linear4",
        "rmsnorm", "post_norm_add", "silu_mul", "embed8", "argmax", "gemv4_rmsnorm", "gemv8_rmsnorm",
        "gemv4_silu", "gemv4_post_norm_add", "gemv4_rmsnorm_silu")
_LIB = ("lib", "check", "MioriError", "OUT_F32", "OUT_BF16", "LAUNCH_PDL", "GEMV_EXACT")

__all__ = list(_OPS + _LIB)


def __getattr__(name):
    if name in _OPS:
        return getattr(importlib.import_module(".ops", __name__), name)
    if name in _LIB:
        return getattr(importlib.import_module("._lib", __name__), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")

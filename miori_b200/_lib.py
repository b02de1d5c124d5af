"""ctypes binding of the C ABI declared in include/miori_b200.h.

There is no fallback: if libmiori_b200.so is missing or a symbol is absent, importing
this module raises.
"""
from __future__ import annotations

import ctypes as C
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
# MIORI_B200_LIB points at another build of the library (A/B comparisons of kernels)
LIB_PATH = os.environ.get("MIORI_B200_LIB") or os.path.join(HERE, "libmiori_b200.so")
HEADER = os.path.join(HERE, "..", "include", "miori_b200.h")

OUT_F32, OUT_BF16, LAUNCH_PDL, GEMV_EXACT = 0, 1, 2, 4

_p, _u32, _sz, _i = C.c_void_p, C.c_uint32, C.c_size_t, C.c_int

_SIGS = {
    "miori_last_error": (C.c_char_p, []),
    "miori_version": (C.c_char_p, []),
    "miori_device_open": (_i, [_i, C.POINTER(_p)]),
    "miori_device_close": (_i, [_p]),
    "miori_device_stream": (_p, [_p]),
    "miori_device_ordinal": (_i, [_p]),
    "miori_buffer_alloc": (_i, [_p, _sz, _i, C.POINTER(_p)]),
    "miori_buffer_free": (_i, [_p]),
    "miori_buffer_contents": (_p, [_p]),
    "miori_buffer_device_ptr": (_p, [_p]),
    "miori_buffer_length": (_sz, [_p]),
    "miori_buffer_prefetch": (_i, [_p, _i]),
    "miori_begin": (_i, [_p]),
    "miori_submit": (_i, [_p, _i]),
    "miori_host_alloc": (_i, [_sz, C.POINTER(_p)]),
    "miori_host_free": (_i, [_p]),
    "miori_memcpy_h2d": (_i, [_p, _p, _sz, _p]),
    "miori_memcpy_d2h": (_i, [_p, _p, _sz, _p]),
    "miori_stream_sync": (_i, [_p]),
    "miori_gemv4": (_i, [_p, _p, _p, _p, _p, _u32, _u32, _u32, _u32, _u32, _p]),
    "miori_gemv8": (_i, [_p, _p, _p, _p, _p, _u32, _u32, _u32, _u32, _u32, _p]),
    "miori_dequant4_rowmajor": (_i, [_p, _p, _p, _p, _u32, _u32, _u32, _p]),
    "miori_dequant8_rowmajor": (_i, [_p, _p, _p, _p, _u32, _u32, _u32, _p]),
    "miori_cache_bytes": (_sz, [_u32, _u32]),
    "miori_dequant4_cache": (_i, [_p, _p, _p, _p, _u32, _u32, _u32, _p]),
    "miori_cache_to_rowmajor": (_i, [_p, _p, _u32, _u32, _p]),
    "miori_gemm_bf16_cache": (_i, [_p, _p, _p, _u32, _u32, _u32, _u32, _p]),
    "miori_gemm_workspace_bytes": (_sz, [_u32, _u32, _u32]),
    "miori_gemm_bf16_cache_ws": (_i, [_p, _p, _p, _u32, _u32, _u32, _u32, _p, _sz, _p]),
    "miori_gemm_static_scratch_bytes": (_sz, []),
    "miori_gemm_bf16_cache_static": (_i, [_p, _p, _p, _u32, _u32, _u32, _u32, _p]),
    "miori_gemm_bf16_strided": (_i, [_p, _u32, _p, _u32, _p, _u32, _u32, _u32, _u32, _u32, _p]),
    "miori_linear4_route": (_i, [_u32, _u32, _u32, _i]),
    "miori_gemv_bf16_cache": (_i, [_p, _p, _p, _u32, _u32, _u32, _u32, _p]),
    "miori_gemm_plan": (_i, [_u32, _u32, _u32, _sz, C.POINTER(_u32), C.POINTER(_u32), C.POINTER(_u32)]),
    "miori_linear4": (_i, [_p, _p, _p, _p, _p, _p, _u32, _u32, _u32, _u32, _u32, _p, _sz, _p]),
    "miori_gemv_argmax_bytes": (_sz, [_i]),
    "miori_gemv4_argmax": (_i, [_p, _p, _p, _p, _p, _sz, _sz, _u32, _u32, _u32, _u32, _u32, _u32, _p]),
    "miori_gemv8_argmax": (_i, [_p, _p, _p, _p, _p, _sz, _sz, _u32, _u32, _u32, _u32, _u32, _u32, _p]),
    "miori_peers_create": (_i, [_i, _i, _sz, C.POINTER(_p)]),
    "miori_peers_handle_bytes": (_sz, []),
    "miori_peers_handle": (_i, [_p, _p]),
    "miori_peers_connect": (_i, [_p, _p]),
    "miori_peers_arena": (_p, [_p]),
    "miori_peers_arena_bytes": (_sz, [_p]),
    "miori_peers_status": (_i, [_p]),
    "miori_peers_set_wait_us": (_i, [_p, _u32]),
    "miori_peers_destroy": (_i, [_p]),
    "miori_gemv4_allgather": (_i, [_p, _p, _p, _p, _p, _sz, _u32, _u32, _u32, _u32, _u32, _u32, _u32, _p]),
    "miori_gemv8_allgather": (_i, [_p, _p, _p, _p, _p, _sz, _u32, _u32, _u32, _u32, _u32, _u32, _u32, _p]),
    "miori_allgather": (_i, [_p, _p, _sz, _u32, _u32, _u32, _u32, _u32, _u32, _p]),
    "miori_argmax_allreduce": (_i, [_p, _p, _u32, _u32, _sz, _u32, _p]),
    "miori_rmsnorm": (_i, [_p, _p, _p, _u32, _u32, C.c_float, _u32, _p]),
    "miori_post_norm_add": (_i, [_p, _p, _p, _p, _u32, _u32, C.c_float, _u32, _p]),
    "miori_silu_mul": (_i, [_p, _p, _p, _sz, _u32, _p]),
    "miori_embed8": (_i, [_p, _p, _p, _p, _p, _u32, _u32, _u32, _u32, _u32, _p]),
    "miori_argmax": (_i, [_p, _u32, _u32, _p, _p, _p]),
    "miori_gemv4_silu": (_i, [_p, _p, _p, _p, _p, _u32, _u32, _u32, _u32, _u32, _p]),
    "miori_gemv4_post_norm_add": (_i, [_p, _p, _p, _p, _p, _p, C.c_float, _p, _p, _u32, _u32, _u32, _u32, _u32, _p]),
    "miori_gemv4_rmsnorm_silu": (_i, [_p, _p, _p, _p, _p, C.c_float, _p, _u32, _u32, _u32, _u32, _u32, _p]),
    "miori_gemv4_rmsnorm": (_i, [_p, _p, _p, _p, _p, C.c_float, _p, _u32, _u32, _u32, _u32, _u32, _p]),
    "miori_gemv8_rmsnorm": (_i, [_p, _p, _p, _p, _p, C.c_float, _p, _u32, _u32, _u32, _u32, _u32, _p]),
    "miori_device_error_poll": (_i, []),
}


def declared_symbols() -> list[str]:
    """Every function name declared in include/miori_b200.h."""
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(miori_[a-z0-9_]+)\s*\(", text)))


class MioriError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"miori_b200 error {code}: {msg}")
        self.code = code


def load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m miori_b200.build` "
            "(there is no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in _SIGS.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is absent
        fn.restype = res
        fn.argtypes = args
    return lib


lib = load()


def check(rc: int) -> None:
    if rc != 0:
        raise MioriError(rc, lib.miori_last_error().decode())

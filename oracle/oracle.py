"""numpy/ctypes front end of the CPU oracle (TEST INFRASTRUCTURE -- never imported by the
product package).  `port` is the plain-C restatement (oracle/miori_oracle.c); `ref` is the
reference's own src/cpu_ref.h compiled by oracle/Makefile into oracle/_ref/ (group 32
only, because that header hard-codes it), or None when it was not built."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_PATH = os.path.join(HERE, "libmiori_oracle.so")
REF_PATH = os.path.join(HERE, "_ref", "libmiori_cpuref.so")

_pp = C.c_void_p
_i64 = C.c_int64


def build() -> None:
    """Compile the oracle (and oracle/_ref when the reference sources are present)."""
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    r = subprocess.run(["make", "-C", HERE], env=env, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + r.stdout + r.stderr)


def _ptr(a: np.ndarray) -> int:
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


def as_u32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a)).view(np.uint32)


def as_u16(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a)).view(np.uint16)


class Port:
    """oracle/miori_oracle.c"""

    def __init__(self):
        if not os.path.exists(PORT_PATH):
            build()
        self.lib = L = C.CDLL(PORT_PATH)
        L.mo_bf16_to_float.restype = C.c_float
        L.mo_bf16_to_float.argtypes = [C.c_uint16]
        L.mo_float_to_bf16.restype = C.c_uint16
        L.mo_float_to_bf16.argtypes = [C.c_float]
        L.mo_bf16_to_float_n.argtypes = [_pp, _pp, C.c_size_t]
        L.mo_float_to_bf16_n.argtypes = [_pp, _pp, C.c_size_t]
        L.mo_dequant_elem.restype = C.c_float
        L.mo_dequant_elem.argtypes = [C.c_int, _pp, _pp, _pp, _i64, _i64, _i64, _i64]
        L.mo_gemv.argtypes = [C.c_int, _pp, _pp, _pp, _pp, _pp, _i64, _i64, _i64, _i64, _i64, _i64]
        L.mo_dequant_rowmajor.argtypes = [C.c_int, _pp, _pp, _pp, _pp, _i64, _i64, _i64]
        L.mo_dequant_tile.argtypes = [_pp, _pp, _pp, _pp, _i64, _i64, _i64]
        L.mo_gemm_bf16.argtypes = [_pp, _pp, _pp, _i64, _i64, _i64, _i64, _i64]
        L.mo_gemm_bf16_entry.restype = C.c_double
        L.mo_gemm_bf16_entry.argtypes = [_pp, _pp, _i64, _i64, _i64]
        L.mo_quantize.argtypes = [C.c_int, _pp, _pp, _pp, _pp, _i64, _i64, _i64]
        L.mo_rmsnorm.argtypes = [_pp, _pp, _pp, _i64, _i64, C.c_float]
        L.mo_silu_mul.argtypes = [_pp, _pp, _pp, _i64]
        L.mo_post_norm_add.argtypes = [_pp, _pp, _pp, _pp, _i64, _i64, C.c_float]
        L.mo_embed8.argtypes = [_pp, _pp, _pp, _pp, _pp, _i64, _i64, _i64]
        L.mo_num_threads.restype = C.c_int
        L.mo_set_threads.argtypes = [C.c_int]

    def threads(self) -> int:
        return self.lib.mo_num_threads()

    def set_threads(self, n: int) -> None:
        self.lib.mo_set_threads(n)

    def bf16_to_float(self, a) -> np.ndarray:
        a = as_u16(a)
        out = np.empty(a.shape, np.float32)
        self.lib.mo_bf16_to_float_n(_ptr(a), _ptr(out), a.size)
        return out

    def float_to_bf16(self, a) -> np.ndarray:
        a = np.ascontiguousarray(a, np.float32)
        out = np.empty(a.shape, np.uint16)
        self.lib.mo_float_to_bf16_n(_ptr(a), _ptr(out), a.size)
        return out

    def dequant_elem(self, bits, q, s, b, n, k, K, group) -> float:
        return self.lib.mo_dequant_elem(bits, _ptr(as_u32(q)), _ptr(as_u16(s)), _ptr(as_u16(b)), n,
                                        k, K, group)

    def gemv(self, bits, q, s, b, x, group, rows=None) -> np.ndarray:
        """y[M][N] in float64; rows=(n0,n1) restricts the computed rows (others are 0)."""
        q, s, b, x = as_u32(q), as_u16(s), as_u16(b), as_u16(x)
        if x.ndim == 1:
            x = x[None, :]
        M, K = x.shape
        N = q.shape[0]
        n0, n1 = rows if rows is not None else (0, N)
        y = np.zeros((M, N), np.float64)
        self.lib.mo_gemv(bits, _ptr(q), _ptr(s), _ptr(b), _ptr(x), _ptr(y), N, K, M, group, n0, n1)
        return y

    def dequant_rowmajor(self, bits, q, s, b, group) -> np.ndarray:
        q, s, b = as_u32(q), as_u16(s), as_u16(b)
        N = q.shape[0]
        K = q.shape[1] * (32 // bits)
        out = np.empty((N, K), np.uint16)
        self.lib.mo_dequant_rowmajor(bits, _ptr(q), _ptr(s), _ptr(b), _ptr(out), N, K, group)
        return out

    def dequant_tile(self, q, s, b, group) -> np.ndarray:
        q, s, b = as_u32(q), as_u16(s), as_u16(b)
        N, K = q.shape[0], q.shape[1] * 8
        out = np.empty((N // 64, K, 64), np.uint16)
        self.lib.mo_dequant_tile(_ptr(q), _ptr(s), _ptr(b), _ptr(out), N, K, group)
        return out

    def gemm_bf16(self, A, Bc, rows=None) -> np.ndarray:
        A, Bc = as_u16(A), as_u16(Bc)
        M, K = A.shape
        N = Bc.shape[0]
        m0, m1 = rows if rows is not None else (0, M)
        Cm = np.zeros((M, N), np.float64)
        self.lib.mo_gemm_bf16(_ptr(A), _ptr(Bc), _ptr(Cm), M, N, K, m0, m1)
        return Cm

    def gemm_entry(self, A, Bc, m, n) -> float:
        A, Bc = as_u16(A), as_u16(Bc)
        return self.lib.mo_gemm_bf16_entry(_ptr(A), _ptr(Bc), A.shape[1], m, n)

    def rmsnorm(self, x, w, eps) -> np.ndarray:
        """bf16 bits of x * rsqrt(mean(x^2) + eps) * w, x [rows][n] fp32, w [n] bf16 bits."""
        x = np.ascontiguousarray(x, np.float32)
        w = as_u16(w)
        y = np.empty(x.shape, np.uint16)
        self.lib.mo_rmsnorm(_ptr(x), _ptr(w), _ptr(y), x.shape[0], x.shape[1], eps)
        return y

    def silu_mul(self, gate, up) -> np.ndarray:
        gate, up = np.ascontiguousarray(gate, np.float32), np.ascontiguousarray(up, np.float32)
        out = np.empty(gate.shape, np.uint16)
        self.lib.mo_silu_mul(_ptr(gate), _ptr(up), _ptr(out), gate.size)
        return out

    def post_norm_add(self, x, src, w, eps) -> np.ndarray:
        x, src = np.ascontiguousarray(x, np.float32), np.ascontiguousarray(src, np.float32)
        w = as_u16(w)
        out = np.empty(x.shape, np.float32)
        self.lib.mo_post_norm_add(_ptr(x), _ptr(src), _ptr(w), _ptr(out), x.shape[0], x.shape[1], eps)
        return out

    def embed8(self, q, s, b, tokens, group) -> np.ndarray:
        q, s, b = as_u32(q), as_u16(s), as_u16(b)
        tokens = np.ascontiguousarray(tokens, np.uint32)
        K = q.shape[1] * 4
        out = np.empty((tokens.size, K), np.uint16)
        self.lib.mo_embed8(_ptr(q), _ptr(s), _ptr(b), _ptr(tokens), _ptr(out), tokens.size, K, group)
        return out

    def quantize(self, bits, W, group):
        W = np.ascontiguousarray(W, np.float32)
        N, K = W.shape
        q = np.empty((N, K * bits // 32), np.uint32)
        s = np.empty((N, K // group), np.uint16)
        b = np.empty((N, K // group), np.uint16)
        self.lib.mo_quantize(bits, _ptr(W), _ptr(q), _ptr(s), _ptr(b), N, K, group)
        return q, s, b


class Ref:
    """oracle/_ref/libmiori_cpuref.so: the reference's src/cpu_ref.h itself (group 32)."""

    def __init__(self):
        self.lib = L = C.CDLL(REF_PATH)
        L.ref_bf16_to_float.restype = C.c_float
        L.ref_bf16_to_float.argtypes = [C.c_uint16]
        L.ref_float_to_bf16.restype = C.c_uint16
        L.ref_float_to_bf16.argtypes = [C.c_float]
        L.ref_dequant_elem.restype = C.c_float
        L.ref_dequant_elem.argtypes = [C.c_int, _pp, _pp, _pp, _i64, _i64, _i64, _i64]
        L.ref_gemv.argtypes = [C.c_int, _pp, _pp, _pp, _pp, _pp, _i64, _i64, _i64, _i64, _i64]
        L.ref_dequant_rowmajor.argtypes = [C.c_int, _pp, _pp, _pp, _pp, _i64, _i64]
        L.ref_num_threads.restype = C.c_int
        L.ref_set_threads.argtypes = [C.c_int]

    def threads(self) -> int:
        return self.lib.ref_num_threads()

    def set_threads(self, n: int) -> None:
        self.lib.ref_set_threads(n)

    def dequant_elem(self, bits, q, s, b, n, k, K) -> float:
        q = as_u32(q)
        return self.lib.ref_dequant_elem(bits, _ptr(q), _ptr(as_u16(s)), _ptr(as_u16(b)),
                                         q.shape[0], n, k, K)

    def gemv(self, bits, q, s, b, x, rows=None) -> np.ndarray:
        q, s, b, x = as_u32(q), as_u16(s), as_u16(b), as_u16(x)
        if x.ndim == 1:
            x = x[None, :]
        M, K = x.shape
        N = q.shape[0]
        n0, n1 = rows if rows is not None else (0, N)
        y = np.zeros((M, N), np.float64)
        self.lib.ref_gemv(bits, _ptr(q), _ptr(s), _ptr(b), _ptr(x), _ptr(y), N, K, M, n0, n1)
        return y

    def dequant_rowmajor(self, bits, q, s, b) -> np.ndarray:
        q, s, b = as_u32(q), as_u16(s), as_u16(b)
        N = q.shape[0]
        K = q.shape[1] * (32 // bits)
        out = np.empty((N, K), np.uint16)
        self.lib.ref_dequant_rowmajor(bits, _ptr(q), _ptr(s), _ptr(b), _ptr(out), N, K)
        return out


_port = None
_ref = None


def port() -> Port:
    global _port
    if _port is None:
        _port = Port()
    return _port


def ref():
    """The compiled reference checker, or None if oracle/_ref was not built."""
    global _ref
    if _ref is None and os.path.exists(REF_PATH):
        _ref = Ref()
    return _ref

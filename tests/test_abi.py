"""CPU tests of the C ABI surface: the library loads, exports every declared symbol, and
rejects bad arguments before touching the GPU."""
import ctypes as C

import pytest

from miori_b200 import _lib
from miori_b200._lib import lib


def test_exports_every_declared_symbol():
    declared = _lib.declared_symbols()
    assert len(declared) >= 25
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/miori_b200.h but not exported"
    # and the binding covers the header, so nothing is callable untyped
    assert set(declared) == set(_lib._SIGS)


def test_version_string():
    assert b"sm_100a" in lib.miori_version()


@pytest.mark.parametrize("fn", ["miori_gemv4", "miori_gemv8"])
def test_gemv_rejects_bad_arguments(fn):
    f = getattr(lib, fn)
    ok = 0x1000  # aligned, never dereferenced: validation fails first
    assert f(None, ok, ok, ok, ok, 16, 64, 1, 32, 0, None) == -1
    assert b"null" in lib.miori_last_error()
    assert f(ok, ok, ok, ok, ok, 16, 64, 1, 48, 0, None) == -1
    assert b"group" in lib.miori_last_error()
    assert f(ok, ok, ok, ok, ok, 16, 96, 1, 64, 0, None) == -1
    assert b"multiple" in lib.miori_last_error()
    assert f(ok, ok, ok, ok, ok, 16, 64, 0, 32, 0, None) == -1
    assert f(ok, ok, ok, ok, ok, 16, 64, 33, 32, 0, None) == -1
    assert b"1..32" in lib.miori_last_error()
    assert f(ok + 4, ok, ok, ok, ok, 16, 64, 1, 32, 0, None) == -1
    assert b"aligned" in lib.miori_last_error()
    assert f(ok, ok, ok, ok, ok, 0, 64, 1, 32, 0, None) == -1


def test_dequant_and_gemm_reject_bad_arguments():
    ok = 0x1000
    assert lib.miori_dequant4_rowmajor(ok, ok, ok, None, 16, 64, 32, None) == -1
    assert lib.miori_dequant8_rowmajor(ok, ok, None, ok, 16, 64, 32, None) == -1
    assert lib.miori_dequant4_cache(ok, ok, ok, ok, 16, 100, 32, None) == -1
    assert lib.miori_gemm_bf16_cache(None, ok, ok, 8, 64, 64, 0, None) == -1
    assert lib.miori_gemm_bf16_cache(ok, ok, ok, 8, 64, 100, 0, None) == -1
    assert lib.miori_gemm_bf16_cache(ok, ok, ok, 0, 64, 64, 0, None) == -1
    assert lib.miori_cache_bytes(64, 128) == 64 * 128 * 2


def test_device_open_reports_failure_without_crashing():
    import torch
    h = C.c_void_p()
    rc = lib.miori_device_open(9999, C.byref(h))
    assert rc != 0 and h.value is None
    assert len(lib.miori_last_error()) > 0
    if not torch.cuda.is_available():
        assert lib.miori_device_open(0, C.byref(h)) != 0
    assert lib.miori_device_open(0, None) == -1


def test_ops_refuse_cpu_tensors():
    import torch
    import miori_b200
    q = torch.zeros((16, 8), dtype=torch.int32)
    s = torch.zeros((16, 2), dtype=torch.bfloat16)
    x = torch.zeros((1, 64), dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="no CPU path"):
        miori_b200.gemv4(q, s, s, x)

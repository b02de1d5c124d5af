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


def test_strided_gemm_and_peer_entries_reject_bad_arguments():
    ok = 0x1000
    # a row pitch shorter than the row, empty shapes, null pointers
    assert lib.miori_gemm_bf16_strided(ok, 56, ok, 64, ok, 64, 8, 64, 64, 0, None) == -1
    assert b"pitch" in lib.miori_last_error()
    assert lib.miori_gemm_bf16_strided(ok, 64, ok, 64, ok, 32, 8, 64, 64, 0, None) == -1
    assert lib.miori_gemm_bf16_strided(ok, 64, None, 64, ok, 64, 8, 64, 64, 0, None) == -1
    assert lib.miori_gemm_bf16_strided(ok, 64, ok, 64, ok, 64, 0, 64, 64, 0, None) == -1
    # peer groups: rank outside the world, too many ranks, arena size not a multiple of 256
    h = C.c_void_p()
    assert lib.miori_peers_create(2, 2, 1 << 20, C.byref(h)) == -1 and h.value is None
    assert lib.miori_peers_create(0, 9, 1 << 20, C.byref(h)) == -1
    assert lib.miori_peers_create(0, 1, 1000, C.byref(h)) == -1
    assert b"256" in lib.miori_last_error()
    assert lib.miori_peers_handle_bytes() == 64
    assert lib.miori_gemv4_allgather(None, ok, ok, ok, ok, 0, 16, 0, 16, 64, 1, 64, 0, None) == -1
    assert lib.miori_allgather(None, ok, 0, 1, 16, 0, 16, 4, 0, None) == -1
    assert lib.miori_peers_status(None) == -1
    assert lib.miori_peers_destroy(None) == 0


def test_neighbor_and_narrow_batch_entries_reject_bad_arguments():
    ok = 0x1000  # aligned, never dereferenced: validation fails first
    assert lib.miori_gemv_bf16_cache(None, ok, ok, 8, 64, 64, 0, None) == -1
    assert b"null" in lib.miori_last_error()
    assert lib.miori_gemv_bf16_cache(ok, ok, ok, 0, 64, 64, 0, None) == -1
    assert lib.miori_gemv_bf16_cache(ok, ok, ok, 33, 64, 64, 0, None) == -1
    assert b"1..32" in lib.miori_last_error()
    assert lib.miori_gemv_bf16_cache(ok, ok, ok, 8, 64, 100, 0, None) == -1
    assert b"multiple of 8" in lib.miori_last_error()
    assert lib.miori_gemv_bf16_cache(ok, ok + 2, ok, 8, 64, 64, 0, None) == -1
    assert b"aligned" in lib.miori_last_error()
    # a K beyond the kernel's range: refused on the host, nothing launched
    assert lib.miori_gemv_bf16_cache(ok, ok, ok, 32, 64, 8192 + 8, 0, None) == -1
    assert b"8192" in lib.miori_last_error()
    # the gated GEMV: N holds the gate rows and then as many up rows, eight of each per tile
    assert lib.miori_gemv4_silu(ok, ok, ok, ok, ok, 24, 64, 1, 32, 0, None) == -1
    assert b"multiple of 16" in lib.miori_last_error()
    assert lib.miori_gemv4_silu(ok, ok, ok, ok, ok, 32, 64, 33, 32, 0, None) == -1
    assert lib.miori_gemv4_silu(ok, ok, ok, None, ok, 32, 64, 1, 32, 0, None) == -1
    assert lib.miori_gemv4_silu(ok, ok, ok, ok, ok, 32, 96, 1, 64, 0, None) == -1
    # the GEMV with the post-norm epilogue: up to four rows, fp32 out, a counter word
    assert lib.miori_gemv4_post_norm_add(ok, ok, ok, ok, ok + 64, ok, 1e-5, ok, ok, 32, 64, 5, 32, 0, None) == -1
    assert b"1..4" in lib.miori_last_error()
    assert lib.miori_gemv4_post_norm_add(ok, ok, ok, ok, ok + 64, ok, 1e-5, None, ok, 32, 64, 1, 32, 0, None) == -1
    assert lib.miori_gemv4_post_norm_add(ok, ok, ok, ok, ok, ok, 1e-5, ok, ok, 32, 64, 1, 32, 0, None) == -1
    assert b"residual" in lib.miori_last_error()
    assert lib.miori_gemv4_post_norm_add(ok, ok, ok, ok, ok + 64, ok, 1e-5, ok, ok, 32, 64, 1, 32, 1, None) == -1
    assert lib.miori_gemv4_rmsnorm_silu(ok, ok, ok, ok, ok, 1e-5, ok, 32, 64, 5, 32, 0, None) == -1
    assert b"1..4" in lib.miori_last_error()
    assert lib.miori_gemv4_rmsnorm_silu(ok, ok, ok, ok, None, 1e-5, ok, 32, 64, 1, 32, 0, None) == -1
    assert lib.miori_gemv4_rmsnorm_silu(ok, ok, ok, ok, ok, 1e-5, ok, 24, 64, 1, 32, 0, None) == -1
    assert lib.miori_rmsnorm(None, ok, ok, 1, 64, 1e-5, 0, None) == -1
    assert lib.miori_rmsnorm(ok, ok, ok, 0, 64, 1e-5, 0, None) == -1
    assert lib.miori_argmax(ok, 0, 0, ok, ok, None) == -1
    assert lib.miori_argmax(None, 8, 0, ok, ok, None) == -1
    # the routing query is pure host arithmetic
    assert lib.miori_linear4_route(4, 2048, 2048, 1) == 0      # up to four rows: packed weights
    assert lib.miori_linear4_route(8, 2048, 2048, 0) == 0      # no cache: packed weights
    assert lib.miori_linear4_route(8, 2048, 2048, 1) == 1      # short projection: narrow-batch cache kernel
    assert lib.miori_linear4_route(8, 16384, 2048, 1) == 0     # wide projection, few rows: packed weights
    assert lib.miori_linear4_route(16, 16384, 2048, 1) == 1
    assert lib.miori_linear4_route(32, 16384, 2048, 1) == 2    # wide and more than 16 rows: tensor-core GEMM
    assert lib.miori_linear4_route(16, 2048, 8192, 1) == 1     # long rows, streamed activations
    assert lib.miori_linear4_route(32, 2048, 8192, 1) == 2     # ... which stops paying above 16 rows

"""The allocation-free split-K GEMM entry (miori_gemm_bf16_cache_static).

It exists for hosts that cannot allocate device memory at call time (a decode loop whose
memory was divided up at start-up, a plug-in under someone else's allocator): the K-split
partials live in a 16 MiB array built into the library instead of a caller workspace.  The
test calls it through the C ABI twice in a row and holds both results to the existing
workspace entry's result with the GEMM tolerance used elsewhere in this suite; the second
call also proves that the scratch left behind by the first does no harm.  Collected last so
that a failure here cannot hide another test's result.
"""
import pytest
import torch

import miori_b200
from miori_b200 import synth
from miori_b200._lib import check, lib
from conftest import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _problem(M, N, K, seed):
    q, s, b = synth.make_weight(N, K, 4, 64, seed=seed, device=DEV)
    cache = miori_b200.dequant4_cache(q, s, b, group=64)
    A = synth.make_activation(M, K, seed=seed + 1, device=DEV)
    return A, cache


def _static(A, cache, N, flags=0):
    M, K = A.shape
    dt = torch.bfloat16 if flags & miori_b200.OUT_BF16 else torch.float32
    out = torch.empty((M, N), dtype=dt, device=DEV)
    check(lib.miori_gemm_bf16_cache_static(A.data_ptr(), cache.data_ptr(), out.data_ptr(), M, N, K,
                                           flags, torch.cuda.current_stream().cuda_stream))
    return out


@pytest.mark.parametrize("M,N,K", [(32, 2048, 2048), (24, 3072, 2048), (32, 2048, 8192)])
def test_static_scratch_matches_workspace_entry_twice(M, N, K):
    A, cache = _problem(M, N, K, seed=M + N + K)
    ws = miori_b200.gemm_workspace(M, N, K, DEV)
    assert ws is not None and ws.numel() * 4 <= lib.miori_gemm_static_scratch_bytes()
    want = miori_b200.gemm_bf16_cache(A, cache, N, workspace=ws)
    first = _static(A, cache, N)
    # a different problem in between leaves other partials in the shared scratch
    A2, cache2 = _problem(16, 512, 1024, seed=5)
    _static(A2, cache2, 512)
    second = _static(A, cache, N)
    torch.cuda.synchronize()
    assert_close(first.cpu().numpy(), want.cpu().numpy(), rel_max=1e-4, what="first static call")
    assert_close(second.cpu().numpy(), want.cpu().numpy(), rel_max=1e-4, what="second static call")
    assert torch.equal(first, second)
    assert lib.miori_device_error_poll() == 0


def test_shape_without_split_runs_and_oversized_split_is_refused():
    A, cache = _problem(300, 256, 128, seed=9)  # too short a K to split: no scratch involved
    assert torch.equal(_static(A, cache, 256), miori_b200.gemm_bf16_cache(A, cache, 256))
    # 1024 x 2304 with a very long K has few tiles for the SMs, so it wants to split K, and two
    # slices of 9 MiB are more than the built-in 16 MiB.  Whether it splits is the planner's
    # decision, so ask first (host-only) and use real operands: if the plan ever changes, the call
    # computes a product instead of being refused -- a failed assertion, never a bad address.
    M, N, K = 1024, 2304, 32768
    if lib.miori_gemm_workspace_bytes(M, N, K) <= lib.miori_gemm_static_scratch_bytes():
        pytest.skip("the planner no longer wants more scratch than the built-in array for this shape")
    A = torch.zeros((M, K), dtype=torch.bfloat16, device=DEV)
    cache = torch.zeros((N, K), dtype=torch.bfloat16, device=DEV)
    out = torch.empty((M, N), dtype=torch.float32, device=DEV)
    rc = lib.miori_gemm_bf16_cache_static(A.data_ptr(), cache.data_ptr(), out.data_ptr(), M, N, K, 0,
                                          torch.cuda.current_stream().cuda_stream)
    assert rc == -1
    msg = lib.miori_last_error().decode()
    assert "scratch" in msg and "miori_gemm_bf16_cache " in msg and str(16 << 20) in msg


def test_static_entry_allocates_nothing():
    """Free device memory is the same before and after a call that uses the built-in scratch."""
    M, N, K = 32, 2048, 2048
    A, cache = _problem(M, N, K, seed=77)
    assert lib.miori_gemm_workspace_bytes(M, N, K) > 0  # the shape does use scratch
    out = torch.empty((M, N), dtype=torch.float32, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    # the first call on a device looks the array's address up; measure around a later one
    check(lib.miori_gemm_bf16_cache_static(A.data_ptr(), cache.data_ptr(), out.data_ptr(), M, N, K, 0, st))
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        check(lib.miori_gemm_bf16_cache_static(A.data_ptr(), cache.data_ptr(), out.data_ptr(), M, N, K, 0, st))
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, f"free device memory changed by {free0 - free1} bytes across the calls"

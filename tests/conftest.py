import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")

# Tolerances of the quantized-matmul path against the CPU oracle.
#   Contract: max|d| <= 1e-2 * max|ref| and cosine >= 0.9999 for every GEMV / GEMM output.
#   The fp32-dequant GEMV (M <= 4) is additionally held to 2e-5 * max|ref|, the order of the
#   reference's own recorded error (max_rel 8.35e-05 on real weights).
TOL_REL_MAX = 1e-2
TOL_COS = 0.9999
TOL_EXACT_PATH = 2e-5


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def port():
    from oracle import oracle
    return oracle.port()


@pytest.fixture(scope="session")
def ref():
    from oracle import oracle
    return oracle.ref()


def u16(t):
    """torch bf16 tensor -> numpy uint16 bits."""
    import torch
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def u32(t):
    return t.detach().cpu().contiguous().numpy().view(np.uint32)


def closeness(got, want):
    """(max|d| / max|ref|, cosine) between two arrays, in float64."""
    g = np.asarray(got, np.float64).ravel()
    w = np.asarray(want, np.float64).ravel()
    scale = max(np.abs(w).max(), 1e-30)
    rel = np.abs(g - w).max() / scale
    den = np.linalg.norm(g) * np.linalg.norm(w)
    cos = float(g @ w / den) if den > 0 else 1.0
    return rel, cos


def assert_close(got, want, rel_max=TOL_REL_MAX, cos_min=TOL_COS, what=""):
    rel, cos = closeness(got, want)
    assert np.isfinite(np.asarray(got, np.float64)).all(), f"{what}: non-finite output"
    assert rel <= rel_max, f"{what}: max|d|/max|ref| = {rel:.3e} > {rel_max:.1e}"
    assert cos >= cos_min, f"{what}: cosine {cos:.7f} < {cos_min}"

"""The cache GEMM's planner against measurement: for every benchmark shape the tile shape and K split
that `plan_gemm` picks (asked through the host-only miori_gemm_plan) must be within 6 % of the
fastest candidate in tests/golden/gemm_candidates.json, a table of CUDA-event timings taken on a
B200 by tests/golden/make_gemm_candidates.py.  No GPU needed: the planner is host arithmetic."""
import ctypes as C
import json
import os

import pytest

from miori_b200._lib import lib

HERE = os.path.dirname(os.path.abspath(__file__))
TABLE = json.load(open(os.path.join(HERE, "golden", "gemm_candidates.json")))["rows"]


def _name(tile_n, ctas, splits):
    return ("256x256 pair" if ctas == 2 else f"128x{tile_n}") + f" x{splits}"


@pytest.mark.parametrize("row", TABLE, ids=lambda r: f"M{r['M']}_N{r['N']}_K{r['K']}")
def test_planner_picks_a_measured_fast_candidate(row):
    M, N, K = row["M"], row["N"], row["K"]
    t, c, s = C.c_uint32(), C.c_uint32(), C.c_uint32()
    assert lib.miori_gemm_plan(M, N, K, 16 * M * N * 4, C.byref(t), C.byref(c), C.byref(s)) == 0
    pick = _name(t.value, c.value, s.value)
    best = min(row["us"].values())
    if pick in row["us"]:
        got = row["us"][pick]
    else:  # a split count the table has no column for: the run of the default plan was timed too
        assert [t.value, c.value, s.value] == row["pick"], "the planner changed: regenerate the table"
        got = row["default_us"]
    assert got <= 1.06 * best, f"M={M} N={N} K={K}: planner picks {pick} ({got} us), fastest measured {best} us"


def test_no_workspace_means_no_split():
    t, c, s = C.c_uint32(), C.c_uint32(), C.c_uint32()
    assert lib.miori_gemm_plan(32, 2048, 8192, 0, C.byref(t), C.byref(c), C.byref(s)) == 0
    assert s.value == 1 and c.value == 1
    assert lib.miori_gemm_plan(0, 2048, 8192, 0, C.byref(t), C.byref(c), C.byref(s)) != 0

"""Build libmiori_b200.so in-tree with nvcc for sm_100a.

The library is one translation unit (csrc/miori_b200.cu) that includes every kernel, so
one nvcc call builds everything.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libmiori_b200.so")
SHIM_LIB = os.path.join(HERE, "libmiori_shim.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "--shared",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _sources(root: str, exts: tuple[str, ...]) -> list[str]:
    out = []
    for d, _, files in os.walk(root):
        out += [os.path.join(d, f) for f in files if f.endswith(exts)]
    return out


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the CUDA library (and the C++ operator shim) if sources are newer."""
    srcs = _sources(CSRC, (".cu", ".cuh", ".h")) + [os.path.join(HERE, "..", "include", "miori_b200.h")]
    if force or _stale(LIB, srcs):
        cmd = [_nvcc(), *NVCC_FLAGS, "-o", LIB, os.path.join(CSRC, "miori_b200.cu")]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
        # nvcc's host compiler must be the PATH gcc (the image's CC lacks a C++ runtime setup)
        env = dict(os.environ)
        env.pop("CC", None)
        env.pop("CXX", None)
        r = subprocess.run(cmd, env=env, capture_output=True, text=True)
        if verbose:
            sys.stderr.write(r.stderr)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + r.stdout + r.stderr)
    shim_dir = os.path.join(HERE, "shim")
    shim_srcs = _sources(shim_dir, (".cpp", ".h", ".hpp"))
    shim_cpp = [s for s in shim_srcs if s.endswith(".cpp")]
    if shim_cpp and (force or _stale(SHIM_LIB, shim_srcs + [LIB])):
        cmd = ["g++", "-std=c++20", "-O2", "-fPIC", "-shared", "-Wall", "-Wextra",
               "-I", shim_dir, "-I", os.path.join(HERE, "..", "include"),
               "-o", SHIM_LIB, *shim_cpp, "-L", HERE, "-lmiori_b200", "-Wl,-rpath,$ORIGIN"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("shim build failed:\n" + r.stdout + r.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))

"""Host-side checks of the C++ operator shim that need no GPU.

1. Error behaviour: shim.cpp is compiled against a fake C ABI (tests/fake_abi/fake_miori.c, host
   memory, scriptable failures) and driven by tests/fake_abi/shim_errors.cpp: a device that cannot
   be opened is reported by Metal::init's return value, everything the reference throws on
   (new_buffer, begin, submit) throws std::runtime_error, and an error recorded by a kernel
   surfaces at the waiting submit.
2. Interface: every operator prototype in shim/ops.h is, token for token, the prototype of the same
   name in the reference's src/ops.h, when the reference sources are mounted beside the repository
   (or MIORI_REFERENCE points at them); parameter names and defaults included.
"""
import os
import re
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SHIM = os.path.join(ROOT, "miori_b200", "shim")


def test_shim_error_paths_against_fake_abi(tmp_path):
    fake_o, exe = str(tmp_path / "fake_miori.o"), str(tmp_path / "shim_errors")
    subprocess.run(["gcc", "-std=gnu11", "-c", os.path.join(HERE, "fake_abi", "fake_miori.c"), "-o", fake_o],
                   check=True)
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", SHIM, "-I", os.path.join(ROOT, "include"),
                    os.path.join(HERE, "fake_abi", "shim_errors.cpp"), os.path.join(SHIM, "shim.cpp"), fake_o,
                    "-o", exe], check=True)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "shim_errors: ok" in r.stdout, r.stdout + r.stderr
    assert "FAILED" not in r.stdout


def _prototypes(text):
    """{name: [normalised prototype, ...]} of the free functions `void name(Metal& m, ...);`."""
    text = re.sub(r"//[^\n]*", "", text)
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    out = {}
    for m in re.finditer(r"\bvoid\s+(\w+)\s*\(\s*(Metal\s*&[^;{]*?)\)\s*;", text, flags=re.S):
        args = re.sub(r"\s+", " ", m.group(2)).strip()
        args = re.sub(r"\s*([,*&=])\s*", r"\1", args)
        out.setdefault(m.group(1), []).append(args)
    return out


def _reference_ops_h():
    for base in (os.environ.get("MIORI_REFERENCE"), os.path.join(ROOT, "..", "reference")):
        if base and os.path.isfile(os.path.join(base, "src", "ops.h")):
            return os.path.join(base, "src", "ops.h")
    return None


def test_prototype_parser():
    got = _prototypes("""
        // a comment with void f(Metal& m);
        void gemv4(Metal& m, MTL::ComputeCommandEncoder* e,
                   const Tensor & q, uint32_t N,   uint32_t boff = 0);
        void helper(int);
    """)
    assert got == {"gemv4": ["Metal&m,MTL::ComputeCommandEncoder*e,const Tensor&q,uint32_t N,uint32_t boff=0"]}


def test_shim_prototypes_equal_the_reference_header():
    ref_h = _reference_ops_h()
    if ref_h is None:
        pytest.skip("reference sources not mounted")
    ours = _prototypes(open(os.path.join(SHIM, "ops.h")).read())
    theirs = _prototypes(open(ref_h).read())
    assert len(ours) >= 19
    missing = sorted(set(ours) - set(theirs))
    assert not missing, f"operators the reference header does not declare: {missing}"
    for name, protos in ours.items():
        for p in protos:
            assert p in theirs[name], f"{name}: shim declares\n  {p}\nreference declares\n  " + "\n  ".join(theirs[name])

"""The binding shown in INTEGRATION.md (one ggml node -> the C ABI, as the drop-in back end does it) must compile against the
reference's own ggml.h / ggml-cuda.h and this library's header: field names, op enums and every argument list are checked
by the compiler.  Skipped where the reference tree is not present."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
from powerinfer_b200 import build as _build

REF = _build.reference_dir() or ""                  # $POWERINFER_REF, or a sibling checkout next to this repository

STAND_INS = r"""
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include "ggml.h"
#include "ggml-cuda.h"
"""


def test_reference_side_shim_compiles_against_the_reference_headers(tmp_path):
    if not REF or not os.path.exists(os.path.join(REF, "ggml-cuda.h")) or shutil.which("g++") is None:
        pytest.skip("reference tree or g++ not present")
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    start = text.index("```cpp") + len("```cpp")
    code = text[start:text.index("```", start)]
    assert "GGML_OP_MUL_MAT_SPARSE" in code and "pi_mul_mat_idx" in code and "pi_axpy" in code
    src = tmp_path / "shim.cpp"
    src.write_text(STAND_INS + code)
    r = subprocess.run(["g++", "-std=c++17", "-fsyntax-only", "-w", "-I", REF, "-I", os.path.join(ROOT, "include"), str(src)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]

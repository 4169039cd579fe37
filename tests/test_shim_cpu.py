"""Syntax check of the C++ binding header (include/ltc_attn_shim.hpp): against stand-ins of the
two reference headers it builds on, and, where the reference checkout is present, against the
reference's own headers -- the shim must compile inside the reference tree unchanged."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA_INC = "/usr/local/cuda/include"
REF_INC = os.path.join(os.environ.get("LTCA_REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference"),
                       "include")


def _check(extra_include):
    cmd = ["g++", "-std=c++17", "-fsyntax-only", "-Wall", "-Werror=return-type",
           "-I", os.path.join(ROOT, "include"), "-I", extra_include, "-I", CUDA_INC,
           os.path.join(ROOT, "tests", "stub", "shim_check.cpp")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]


@pytest.mark.skipif(shutil.which("g++") is None or not os.path.isdir(CUDA_INC), reason="needs g++ and CUDA headers")
def test_shim_compiles_against_stand_in_headers():
    _check(os.path.join(ROOT, "tests", "stub"))


@pytest.mark.skipif(shutil.which("g++") is None or not os.path.isdir(CUDA_INC) or
                    not os.path.exists(os.path.join(REF_INC, "time_self_attention.h")),
                    reason="reference checkout not present")
def test_shim_compiles_against_the_reference_headers():
    _check(REF_INC)

"""CPU checks of the drop-in boundary: the library loads without a GPU, exports every symbol
the header declares, and refuses to create a context where no sm_100 device exists."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ltc_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ltca_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from cuda_ltc_b200.build import build_library
    build_library()
    from cuda_ltc_b200 import _lib
    return _lib.load()


def test_header_symbols_are_exported(lib):
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in ltc_attn.h but not exported"


def test_binding_covers_header(lib):
    from cuda_ltc_b200 import _lib
    assert set(declared_symbols()) == set(_lib.EXPORTS)


def test_version(lib):
    assert lib.ltca_version() == 100


def test_struct_sizes_match_header():
    """ctypes mirrors of the parameter blocks must agree with the C compiler's layout."""
    import subprocess, tempfile, textwrap
    from cuda_ltc_b200 import _lib
    src = textwrap.dedent("""
        #include <stdio.h>
        #include "ltc_attn.h"
        int main(void) { printf("%zu %zu %zu\\n", sizeof(ltca_attn_params), sizeof(ltca_tsa_params), sizeof(ltca_strides)); return 0; }
    """)
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "s.c")
        open(c, "w").write(src)
        exe = os.path.join(d, "s")
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe])
        a, t, s = map(int, subprocess.check_output([exe]).split())
    assert (a, t, s) == (C.sizeof(_lib.AttnParams), C.sizeof(_lib.TsaParams), C.sizeof(_lib.Strides))


def test_no_context_without_gpu(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    rc = lib.ltca_ctx_create(0, None, C.byref(h))
    assert rc < 0 and not h.value          # fails loudly; there is no CPU fallback


def test_size_queries_run_without_gpu(lib):
    from cuda_ltc_b200 import _lib
    p = _lib.AttnParams()
    p.B, p.H, p.Sq, p.Sk, p.D = 8, 16, 4096, 4096, 64
    p.dtype, p.mode, p.scale = _lib.LTCA_F32, _lib.MODE_AUTO, 0.125
    n = C.c_size_t(0)
    assert lib.ltca_attn_workspace_bytes(C.byref(p), 0, C.byref(n)) == 0
    assert n.value == 3 * 8 * 16 * 4096 * 64 * 2      # bf16 copies of q, k, v
    p.dtype = _lib.LTCA_BF16
    assert lib.ltca_attn_workspace_bytes(C.byref(p), 0, C.byref(n)) == 0 and n.value == 0
    assert lib.ltca_attn_uses_tensor_pipe(C.byref(p), 0) == 1
    p.D = 32
    assert lib.ltca_attn_uses_tensor_pipe(C.byref(p), 0) == 0


def test_decode_size_query_and_static_entry_reject_bad_shapes_on_the_host(lib):
    """Argument checks run before anything touches a device: no GPU is needed to see the status codes (a zero
    batch x heads used to reach a division in the split planner)."""
    from cuda_ltc_b200 import _lib
    n = C.c_size_t(7)
    err = C.create_string_buffer(200)
    dummy = (C.c_float * 64)()
    for B, H, Sk, D in ((0, 8, 128, 64), (4, 0, 128, 64), (4, -2, 128, 64), (4, 8, 0, 64), (4, 8, 128, 0)):
        p = _lib.AttnParams()
        p.B, p.H, p.Sq, p.Sk, p.D = B, H, 1, Sk, D
        p.dtype, p.mode, p.scale = _lib.LTCA_F32, _lib.MODE_FP32, 0.125
        p.q = p.k = p.v = p.o = C.addressof(dummy)          # never dereferenced: the shape is refused first
        assert lib.ltca_attn_decode_workspace_bytes(C.byref(p), C.byref(n)) == 0 and n.value == 0
        assert lib.ltca_attn_decode_static(None, C.byref(p), err, len(err)) == -1
        assert b"bad decode arguments" in err.value
    assert lib.ltca_attn_decode_static(None, None, err, len(err)) == -1

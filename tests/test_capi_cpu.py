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


def test_mode_and_block_size_queries_without_gpu(lib):
    """Which path a call will take and how much scratch it needs are host-side decisions: the split-precision
    mode takes the written-out-score path at every head width, with two bf16 terms of every operand in its
    workspace; the module's kept-forward and weight-copy blocks follow its pipeline."""
    from cuda_ltc_b200 import _lib
    al = lambda x: (x + 255) // 256 * 256
    p = _lib.AttnParams()
    p.B, p.H, p.Sq, p.Sk, p.D = 2, 4, 64, 64, 32
    p.dtype, p.scale = _lib.LTCA_F32, 32 ** -0.5
    for st in (p.q_strides, p.k_strides, p.v_strides, p.o_strides, p.do_strides, p.dq_strides, p.dk_strides,
               p.dv_strides):
        st.batch, st.head, st.seq = 4 * 64 * 32, 64 * 32, 32
    n = C.c_size_t(0)
    p.mode = _lib.MODE_AUTO
    assert lib.ltca_attn_uses_tensor_pipe(C.byref(p), 0) == 0              # width 32: the exact kernels
    for mode, terms in ((_lib.MODE_BF16, 1), (_lib.MODE_SPLIT, 2)):
        p.mode = mode
        assert lib.ltca_attn_uses_tensor_pipe(C.byref(p), 0) == 1 and lib.ltca_attn_uses_tensor_pipe(C.byref(p), 1) == 1
        packed = al(2 * 4 * 64 * 32 * 2)
        scores = 2 * 4 * 64 * 64
        want_fwd = 3 * packed * terms + al(scores * 4) + 2 * al(scores * 2)
        assert lib.ltca_attn_workspace_bytes(C.byref(p), 0, C.byref(n)) == 0 and n.value == want_fwd
        assert lib.ltca_attn_workspace_bytes(C.byref(p), 1, C.byref(n)) == 0
        assert n.value == want_fwd + packed * terms + al(scores * 4)
    p.D, p.mode = 64, _lib.MODE_SPLIT                                        # the split mode also at width 64 ...
    for st in (p.q_strides, p.k_strides, p.v_strides, p.o_strides):
        st.batch, st.head, st.seq = 4 * 64 * 64, 64 * 64, 64
    assert lib.ltca_attn_workspace_bytes(C.byref(p), 0, C.byref(n)) == 0 and n.value > 6 * al(2 * 4 * 64 * 64 * 2)
    p.dtype = _lib.LTCA_BF16                                                 # ... but with bf16 storage it is the bf16 mode
    assert lib.ltca_attn_workspace_bytes(C.byref(p), 0, C.byref(n)) == 0 and n.value == 0

    t = _lib.TsaParams()
    t.B, t.S, t.E, t.H, t.head_width, t.scale, t.mode = 4, 32, 128, 2, 64, 0.125, _lib.MODE_AUTO
    w_in, w_out = al(128 * 128 * 2), al(128 * 128 * 2)
    assert lib.ltca_tsa_weight_cache_bytes(C.byref(t), C.byref(n)) == 0 and n.value == 3 * w_in + w_out
    t.head_width, t.scale = 128, 1.0                                         # the reference's form at width 128 ...
    assert lib.ltca_tsa_weight_cache_bytes(C.byref(t), C.byref(n)) == 0 and n.value == 0      # ... is exact under AUTO
    t.mode = _lib.MODE_BF16                                                  # on request: written-out scores, Wq and Wk in two terms
    w_in = al(128 * 256 * 2)
    assert lib.ltca_tsa_weight_cache_bytes(C.byref(t), C.byref(n)) == 0 and n.value == 5 * w_in + al(256 * 128 * 2)
    m = C.c_size_t(0)
    assert lib.ltca_tsa_saved_bytes(C.byref(t), C.byref(m)) == 0 and m.value > n.value
    t.mode = _lib.MODE_FP32
    assert lib.ltca_tsa_weight_cache_bytes(C.byref(t), C.byref(n)) == 0 and n.value == 0


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

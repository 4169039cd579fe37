"""The allocation-free decode entry point (ltca_attn_decode_static) against the regular one.

Collected last on purpose (file name): a run that stops at the first failure has then already
exercised every other test.  The entry point serves callers that cannot allocate device memory
(plug-ins inside another framework's arena, loops that ban allocations after start-up): it
takes no context and keeps the split-over-keys partial results in an array built into the
library.  Two calls in a row with different inputs check that what the first call left in the
shared array does not leak into the second.
"""
import ctypes as C
import math

import numpy as np
import pytest
import torch

import oracle
from cuda_ltc_b200 import _lib
from util import randn

pytestmark = pytest.mark.gpu


def _call_static(lib, ctx, q, k, v, kv_len, scale):
    B, H, _, D = q.shape
    o = torch.full((B, H, 1, D), float("nan"), dtype=q.dtype, device=q.device)
    lse = torch.full((B, H, 1), float("nan"), dtype=torch.float32, device=q.device)
    p = ctx._params(q, k, v, o, lse, scale, False, None, kv_len, 0.0, _lib.MODE_FP32)
    err = C.create_string_buffer(256)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.ltca_attn_decode_static(stream, C.byref(p), err, len(err))
    return rc, err.value.decode(), o, lse


def test_static_decode_matches_regular_entry_point(ctx):
    lib = _lib.load()
    B, H, Smax, D = 2, 2, 2048, 128          # few (batch, head) pairs: the key range is split
    scale = 1.0 / math.sqrt(D)
    need = C.c_size_t(0)
    for call, seed in enumerate((900, 901)):
        q, k, v = (torch.from_numpy(randn(s, seed + i)).cuda()
                   for i, s in enumerate(((B, H, 1, D), (B, H, Smax, D), (B, H, Smax, D))))
        kv_len = torch.tensor([Smax, 700 + 300 * call], dtype=torch.int32, device="cuda")
        o_ref, lse_ref = ctx.attn_decode(q, k, v, kv_len=kv_len, scale=scale)
        rc, msg, o, lse = _call_static(lib, ctx, q, k, v, kv_len, scale)
        assert rc == 0, msg
        torch.cuda.synchronize()
        if call == 0:
            p = ctx._params(q, k, v, o, lse, scale, False, None, kv_len, 0.0, _lib.MODE_FP32)
            lib.ltca_attn_decode_workspace_bytes(C.byref(p), C.byref(need))
            assert need.value > 0, "this shape must exercise the scratch path"
        assert np.abs(o.cpu().numpy() - o_ref.cpu().numpy()).max() < 1e-5
        assert np.abs(lse.cpu().numpy() - lse_ref.cpu().numpy()).max() < 1e-5
        # and against the fp64 oracle, so that the pair of entry points cannot be wrong together
        o_orc, lse_orc = oracle.attn_fwd(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy(), scale, False, None,
                                         kv_len.cpu().numpy())
        assert np.abs(o.cpu().numpy() - o_orc).max() < 1e-5
        assert np.abs(lse.cpu().numpy() - lse_orc).max() < 1e-5


def test_static_decode_refuses_oversized_scratch(ctx):
    lib = _lib.load()
    B, H, Smax, D = 50, 4, 16384, 128         # 200 pairs x 3 splits x 130 floats > 256 KiB
    q = torch.zeros((B, H, 1, D), device="cuda")
    k = torch.zeros((B, H, 8, D), device="cuda").expand(B, H, 8, D)
    o = torch.empty_like(q)
    p = ctx._params(q, k, k, o, None, 0.1, False, None, None, 0.0, _lib.MODE_FP32)
    p.Sk = Smax                                 # only the size check runs; nothing is launched
    need = C.c_size_t(0)
    lib.ltca_attn_decode_workspace_bytes(C.byref(p), C.byref(need))
    assert need.value > 256 << 10
    err = C.create_string_buffer(256)
    rc = lib.ltca_attn_decode_static(None, C.byref(p), err, len(err))
    assert rc == -4 and b"262144" in err.value


def test_static_decode_argument_errors_come_back_as_status_codes(ctx):
    """Shapes that are not positive, or a query length other than 1, are refused before any size is computed
    from them (a zero batch x heads once divided by zero in the split planner)."""
    lib = _lib.load()
    q = torch.zeros((2, 2, 1, 64), device="cuda")
    k = torch.zeros((2, 2, 16, 64), device="cuda")
    o = torch.empty_like(q)
    err = C.create_string_buffer(256)
    need = C.c_size_t(123)
    for field, value in (("B", 0), ("H", 0), ("H", -3), ("Sk", 0), ("D", 0), ("Sq", 2)):
        p = ctx._params(q, k, k, o, None, 0.1, False, None, None, 0.0, _lib.MODE_FP32)
        setattr(p, field, value)
        assert lib.ltca_attn_decode_workspace_bytes(C.byref(p), C.byref(need)) == 0
        if field != "Sq":
            assert need.value == 0
        assert lib.ltca_attn_decode_static(None, C.byref(p), err, len(err)) == -1, (field, value)
        assert err.value

"""ctypes binding of libltc_attn.so (the C-ABI library declared in include/ltc_attn.h).

The library is the product; there is no Python or CPU fallback.  Loading fails loudly when the
shared object is missing -- build it with ``python -m cuda_ltc_b200.build``.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libltc_attn.so")

LTCA_F32, LTCA_BF16 = 0, 1
MODE_AUTO, MODE_BF16, MODE_SPLIT, MODE_FP32 = 0, 1, 2, 3

STATUS_NAMES = {
    0: "LTCA_OK", -1: "LTCA_ERR_INVALID", -2: "LTCA_ERR_UNSUPPORTED", -3: "LTCA_ERR_CUDA",
    -4: "LTCA_ERR_WORKSPACE", -5: "LTCA_ERR_DEVICE", -6: "LTCA_ERR_NO_DEVICE",
}


class Strides(C.Structure):
    _fields_ = [("batch", C.c_int64), ("head", C.c_int64), ("seq", C.c_int64)]


class AttnParams(C.Structure):
    _fields_ = [
        ("B", C.c_int32), ("H", C.c_int32), ("Sq", C.c_int32), ("Sk", C.c_int32), ("D", C.c_int32),
        ("dtype", C.c_int32), ("mode", C.c_int32), ("causal", C.c_int32),
        ("scale", C.c_float), ("score_clamp", C.c_float),
        ("q", C.c_void_p), ("q_strides", Strides),
        ("k", C.c_void_p), ("k_strides", Strides),
        ("v", C.c_void_p), ("v_strides", Strides),
        ("o", C.c_void_p), ("o_strides", Strides),
        ("lse", C.c_void_p),
        ("keep_mask", C.c_void_p), ("kv_len", C.c_void_p),
        ("dout", C.c_void_p), ("do_strides", Strides),
        ("dq", C.c_void_p), ("dq_strides", Strides),
        ("dk", C.c_void_p), ("dk_strides", Strides),
        ("dv", C.c_void_p), ("dv_strides", Strides),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("bwd_deterministic", C.c_int32),
    ]


class TsaParams(C.Structure):
    _fields_ = [
        ("B", C.c_int32), ("S", C.c_int32), ("E", C.c_int32), ("H", C.c_int32),
        ("head_width", C.c_int32), ("causal", C.c_int32), ("time_major", C.c_int32),
        ("use_residual", C.c_int32), ("use_layer_norm", C.c_int32), ("mode", C.c_int32),
        ("scale", C.c_float), ("score_clamp", C.c_float),
        ("x", C.c_void_p),
        ("wq", C.c_void_p), ("wk", C.c_void_p), ("wv", C.c_void_p), ("wo", C.c_void_p),
        ("bq", C.c_void_p), ("bk", C.c_void_p), ("bv", C.c_void_p), ("bo", C.c_void_p),
        ("ln_gamma", C.c_void_p), ("ln_beta", C.c_void_p),
        ("keep_mask", C.c_void_p), ("kv_len", C.c_void_p),
        ("out", C.c_void_p),
        ("dy", C.c_void_p), ("dx", C.c_void_p),
        ("dwq", C.c_void_p), ("dwk", C.c_void_p), ("dwv", C.c_void_p), ("dwo", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("pre_norm", C.c_int32), ("dropout_prob", C.c_float), ("dropout_seed", C.c_uint64),
        ("dbq", C.c_void_p), ("dbk", C.c_void_p), ("dbv", C.c_void_p), ("dbo", C.c_void_p),
        ("dgamma", C.c_void_p), ("dbeta", C.c_void_p),
        ("saved", C.c_void_p), ("saved_bytes", C.c_size_t), ("reuse_forward", C.c_int32),
        ("weight_cache", C.c_void_p), ("weight_cache_bytes", C.c_size_t), ("weight_cache_valid", C.c_int32),
    ]


# Every symbol include/ltc_attn.h declares, with its ctypes signature.
EXPORTS = {
    "ltca_version": (C.c_int, []),
    "ltca_ctx_create": (C.c_int, [C.c_int, C.c_void_p, C.POINTER(C.c_void_p)]),
    "ltca_ctx_set_stream": (C.c_int, [C.c_void_p, C.c_void_p]),
    "ltca_ctx_enable_kernel_timing": (C.c_int, [C.c_void_p, C.c_int]),
    "ltca_ctx_last_bwd_kernel_ms": (C.c_int, [C.c_void_p, C.POINTER(C.c_float)]),
    "ltca_ctx_destroy": (None, [C.c_void_p]),
    "ltca_last_error": (C.c_char_p, [C.c_void_p]),
    "ltca_ctx_set_sm_limit": (C.c_int, [C.c_void_p, C.c_int32]),
    "ltca_device_status": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32)]),
    "ltca_selftest_bounded_wait": (C.c_int, [C.c_void_p, C.c_uint32]),
    "ltca_attn_workspace_bytes": (C.c_int, [C.POINTER(AttnParams), C.c_int, C.POINTER(C.c_size_t)]),
    "ltca_attn_uses_tensor_pipe": (C.c_int, [C.POINTER(AttnParams), C.c_int]),
    "ltca_attn_fwd": (C.c_int, [C.c_void_p, C.POINTER(AttnParams)]),
    "ltca_attn_bwd": (C.c_int, [C.c_void_p, C.POINTER(AttnParams)]),
    "ltca_attn_decode": (C.c_int, [C.c_void_p, C.POINTER(AttnParams)]),
    "ltca_attn_decode_workspace_bytes": (C.c_int, [C.POINTER(AttnParams), C.POINTER(C.c_size_t)]),
    "ltca_attn_decode_static": (C.c_int, [C.c_void_p, C.POINTER(AttnParams), C.c_char_p, C.c_size_t]),
    "ltca_tsa_bwd": (C.c_int, [C.c_void_p, C.POINTER(TsaParams)]),
    "ltca_tsa_saved_bytes": (C.c_int, [C.POINTER(TsaParams), C.POINTER(C.c_size_t)]),
    "ltca_tsa_weight_cache_bytes": (C.c_int, [C.POINTER(TsaParams), C.POINTER(C.c_size_t)]),
    "ltca_tsa_workspace_bytes": (C.c_int, [C.POINTER(TsaParams), C.c_int, C.POINTER(C.c_size_t)]),
    "ltca_tsa_fwd": (C.c_int, [C.c_void_p, C.POINTER(TsaParams)]),
    "ltca_tsa_bwd_data": (C.c_int, [C.c_void_p, C.POINTER(TsaParams)]),
    "ltca_tsa_bwd_weights": (C.c_int, [C.c_void_p, C.POINTER(TsaParams)]),
    "ltca_add_tensors": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "ltca_attn_merge": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
                                  C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "ltca_accumulate_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int32,
                                       C.c_int32, C.c_int32, C.c_int32]),
    "ltca_layer_norm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32]),
    "ltca_validate_finite": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "ltca_f32_to_bf16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "ltca_bf16_to_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
}

_lib = None


def load() -> C.CDLL:
    """Loads the library once and attaches the signatures.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: the CUDA library has not been built "
                "(python -m cuda_ltc_b200.build); there is no fallback path")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in EXPORTS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib

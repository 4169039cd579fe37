"""torch-tensor front end over the C ABI (used by tests, smoke check and benchmark).

torch is plumbing here: it owns device memory and streams.  Every function fills an
``ltca_attn_params`` block with raw pointers and strides and calls libltc_attn.so; nothing is
computed in Python and nothing falls back to torch operators.

Tensor convention: ``[batch, heads, seq, head_dim]`` views with ``head_dim`` contiguous (any
batch/head/seq strides), float32 or bfloat16 -- e.g. ``x.view(B, S, H, D).transpose(1, 2)``
addresses an un-permuted ``[B*S, H*D]`` projection output directly.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import AttnParams, Strides


class LtcaError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"{_lib.STATUS_NAMES.get(code, code)}: {message}")
        self.code = code


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _lib.LTCA_F32
    if t.dtype == torch.bfloat16:
        return _lib.LTCA_BF16
    raise TypeError(f"unsupported dtype {t.dtype}")


def _strides(t: torch.Tensor) -> Strides:
    assert t.dim() == 4 and (t.stride(3) == 1 or t.shape[3] == 1), "head_dim must be contiguous"
    return Strides(t.stride(0), t.stride(1), t.stride(2))


class Context:
    """One (device, stream) binding of the library."""

    def __init__(self, device: int = 0, stream: Optional[torch.cuda.Stream] = None):
        self.lib = _lib.load()
        self.device = int(device)
        handle = C.c_void_p()
        sptr = C.c_void_p(stream.cuda_stream) if stream is not None else C.c_void_p(
            torch.cuda.current_stream(self.device).cuda_stream)
        rc = self.lib.ltca_ctx_create(self.device, sptr, C.byref(handle))
        if rc != 0:
            raise LtcaError(rc, "ltca_ctx_create failed (is this an sm_100 GPU?)")
        self.handle = handle
        self._ws = None

    def close(self):
        if getattr(self, "handle", None):
            self.lib.ltca_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_stream(self, stream: torch.cuda.Stream):
        self.lib.ltca_ctx_set_stream(self.handle, C.c_void_p(stream.cuda_stream))

    def enable_kernel_timing(self, enable: bool = True):
        """Per-kernel CUDA-event timing of the tensor-pipe backward (benchmark aid)."""
        self.check(self.lib.ltca_ctx_enable_kernel_timing(self.handle, int(enable)))

    def last_bwd_kernel_ms(self):
        """(statistics, dQ kernel, dK/dV kernel) durations in ms of the last timed backward."""
        ms = (C.c_float * 3)()
        self.check(self.lib.ltca_ctx_last_bwd_kernel_ms(self.handle, ms))
        return tuple(float(x) for x in ms)

    def check(self, rc: int):
        if rc != 0:
            raise LtcaError(rc, self.lib.ltca_last_error(self.handle).decode())

    def set_sm_limit(self, n_sms: int = 0):
        """Cap the SMs the persistent kernels spread over (0 = all): leaves room for a communication
        library's kernels to run beside them."""
        self.check(self.lib.ltca_ctx_set_sm_limit(self.handle, int(n_sms)))

    def sm_count(self) -> int:
        return torch.cuda.get_device_properties(self.device).multi_processor_count

    def device_status(self) -> int:
        v = C.c_uint32(0)
        self.lib.ltca_device_status(self.handle, C.byref(v))
        return int(v.value)

    def selftest_bounded_wait(self, limit_us: int = 20000):
        """Launches the wait self-test: one warp waits `limit_us` for a barrier that never completes, gives up
        and sets the time-out bit that :meth:`device_status` then returns."""
        self.check(self.lib.ltca_selftest_bounded_wait(self.handle, int(limit_us)))

    # ---- small tensor helpers on the path ------------------------------------------------------
    def add_tensors(self, a, b, out=None):
        """out = a + b for fp32 tensors of equal size (the reference's addTensors)."""
        assert a.dtype == b.dtype == torch.float32 and a.numel() == b.numel()
        out = torch.empty_like(a) if out is None else out
        self.check(self.lib.ltca_add_tensors(self.handle, a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel()))
        return out

    def validate_finite(self, x) -> bool:
        """True if every element of the fp32 tensor is finite (the reference's validateGradients)."""
        assert x.dtype == torch.float32
        flag = torch.zeros(1, dtype=torch.int32, device=x.device)
        self.check(self.lib.ltca_validate_finite(self.handle, x.data_ptr(), x.numel(), flag.data_ptr()))
        return int(flag.item()) == 0

    def layer_norm_(self, x, gamma=None, beta=None):
        """In-place LayerNorm of a contiguous fp32 [rows, E] tensor (biased variance, eps 1e-5)."""
        assert x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2
        self.check(self.lib.ltca_layer_norm(self.handle, x.data_ptr(),
                                            gamma.data_ptr() if gamma is not None else None,
                                            beta.data_ptr() if beta is not None else None, x.shape[0], x.shape[1]))
        return x

    def to_bf16(self, x):
        assert x.dtype == torch.float32 and x.is_contiguous()
        out = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
        self.check(self.lib.ltca_f32_to_bf16(self.handle, x.data_ptr(), out.data_ptr(), x.numel()))
        return out

    def to_f32(self, x):
        assert x.dtype == torch.bfloat16 and x.is_contiguous()
        out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        self.check(self.lib.ltca_bf16_to_f32(self.handle, x.data_ptr(), out.data_ptr(), x.numel()))
        return out

    def workspace(self, nbytes: int) -> Optional[torch.Tensor]:
        """A cached scratch buffer of at least ``nbytes`` (grown on demand, 256-byte aligned)."""
        if nbytes == 0:
            return None
        if self._ws is None or self._ws.numel() < nbytes:
            self._ws = torch.empty(nbytes, dtype=torch.uint8, device=f"cuda:{self.device}")
        return self._ws

    # ---- parameter block -----------------------------------------------------------------
    def _params(self, q, k, v, o, lse, scale, causal, keep_mask, kv_len, score_clamp, mode) -> AttnParams:
        B, H, Sq, D = q.shape
        Sk = k.shape[2]
        assert k.shape == (B, H, Sk, D) and v.shape == (B, H, Sk, D) and o.shape == (B, H, Sq, D)
        assert q.dtype == k.dtype == v.dtype == o.dtype
        p = AttnParams()
        p.B, p.H, p.Sq, p.Sk, p.D = B, H, Sq, Sk, D
        p.dtype, p.mode, p.causal = _dtype_code(q), int(mode), int(bool(causal))
        p.scale, p.score_clamp = float(scale), float(score_clamp or 0.0)
        p.q, p.q_strides = q.data_ptr(), _strides(q)
        p.k, p.k_strides = k.data_ptr(), _strides(k)
        p.v, p.v_strides = v.data_ptr(), _strides(v)
        p.o, p.o_strides = o.data_ptr(), _strides(o)
        p.lse = lse.data_ptr() if lse is not None else None
        if keep_mask is not None:
            assert keep_mask.dtype == torch.float32 and keep_mask.is_contiguous()
            assert keep_mask.shape == (B, Sq, Sk)
            p.keep_mask = keep_mask.data_ptr()
        if kv_len is not None:
            assert kv_len.dtype == torch.int32 and kv_len.is_contiguous() and kv_len.shape == (B,)
            p.kv_len = kv_len.data_ptr()
        return p

    def _attach_workspace(self, p: AttnParams, backward: int, fixed: Optional[int] = None):
        need = C.c_size_t(0)
        if fixed is None:
            self.lib.ltca_attn_workspace_bytes(C.byref(p), backward, C.byref(need))
            n = need.value
        else:
            n = fixed
        ws = self.workspace(n)
        if ws is not None:
            p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
        return ws

    # ---- calls ---------------------------------------------------------------------------
    def attn_fwd(self, q, k, v, scale=None, causal=False, keep_mask=None, kv_len=None,
                 score_clamp=0.0, mode=_lib.MODE_AUTO, out=None, lse=None
                 ) -> Tuple[torch.Tensor, torch.Tensor]:
        B, H, Sq, D = q.shape
        scale = 1.0 / math.sqrt(D) if scale is None else scale
        o = torch.empty((B, H, Sq, D), dtype=q.dtype, device=q.device) if out is None else out
        lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device) if lse is None else lse
        p = self._params(q, k, v, o, lse, scale, causal, keep_mask, kv_len, score_clamp, mode)
        ws = self._attach_workspace(p, 0)
        self.check(self.lib.ltca_attn_fwd(self.handle, C.byref(p)))
        del ws
        return o, lse

    def attn_bwd(self, q, k, v, o, lse, dout, scale=None, causal=False, keep_mask=None,
                 kv_len=None, score_clamp=0.0, mode=_lib.MODE_AUTO, dq=None, dk=None, dv=None,
                 deterministic=False):
        """dq, dk, dv.  ``deterministic=True`` asks for bit-identical results from run to run (bf16 storage on the
        tensor pipe otherwise takes the fused kernel, whose dq can differ between runs by fp32 rounding)."""
        D = q.shape[3]
        scale = 1.0 / math.sqrt(D) if scale is None else scale
        dq = torch.empty(q.shape, dtype=q.dtype, device=q.device) if dq is None else dq
        dk = torch.empty(k.shape, dtype=k.dtype, device=k.device) if dk is None else dk
        dv = torch.empty(v.shape, dtype=v.dtype, device=v.device) if dv is None else dv
        p = self._params(q, k, v, o, lse, scale, causal, keep_mask, kv_len, score_clamp, mode)
        p.bwd_deterministic = int(bool(deterministic))
        p.dout, p.do_strides = dout.data_ptr(), _strides(dout)
        p.dq, p.dq_strides = dq.data_ptr(), _strides(dq)
        p.dk, p.dk_strides = dk.data_ptr(), _strides(dk)
        p.dv, p.dv_strides = dv.data_ptr(), _strides(dv)
        ws = self._attach_workspace(p, 1)
        self.check(self.lib.ltca_attn_bwd(self.handle, C.byref(p)))
        del ws
        return dq, dk, dv

    def attn_decode(self, q, k, v, kv_len=None, scale=None, keep_mask=None, score_clamp=0.0,
                    out=None, lse=None):
        B, H, Sq, D = q.shape
        scale = 1.0 / math.sqrt(D) if scale is None else scale
        o = torch.empty((B, H, 1, D), dtype=q.dtype, device=q.device) if out is None else out
        lse = torch.empty((B, H, 1), dtype=torch.float32, device=q.device) if lse is None else lse
        p = self._params(q, k, v, o, lse, scale, False, keep_mask, kv_len, score_clamp, _lib.MODE_FP32)
        need = C.c_size_t(0)
        self.lib.ltca_attn_decode_workspace_bytes(C.byref(p), C.byref(need))
        ws = self._attach_workspace(p, 0, fixed=need.value)
        self.check(self.lib.ltca_attn_decode(self.handle, C.byref(p)))
        del ws
        return o, lse

    # ---- sequence sharding: fold one key/value shard's result into running accumulators ----
    def attn_merge(self, o_acc, lse_acc, o_blk, lse_blk, s0=0):
        """o_acc [B,H,S,D] fp32, lse_acc [B,H,S] fp32 (contiguous) absorb o_blk [B,H,n,D], lse_blk [B,H,n]
        (contiguous) at rows s0 .. s0+n of every (batch, head)."""
        B, H, S, D = o_acc.shape
        n = o_blk.shape[2]
        assert o_acc.is_contiguous() and lse_acc.is_contiguous() and o_blk.is_contiguous() and lse_blk.is_contiguous()
        assert o_acc.dtype == torch.float32 and lse_acc.dtype == torch.float32 and lse_blk.dtype == torch.float32
        self.check(self.lib.ltca_attn_merge(self.handle, o_acc.data_ptr(), lse_acc.data_ptr(), o_blk.data_ptr(),
                                            _dtype_code(o_blk), lse_blk.data_ptr(), B * H, S, s0, n, D))

    def accumulate_rows(self, acc, part, s0=0):
        """acc [B,H,S,D] fp32 += part [B,H,n,D] (fp32 or bf16, contiguous) at rows s0 .. s0+n."""
        B, H, S, D = acc.shape
        assert acc.is_contiguous() and part.is_contiguous() and acc.dtype == torch.float32
        self.check(self.lib.ltca_accumulate_rows(self.handle, acc.data_ptr(), part.data_ptr(), _dtype_code(part),
                                                 B * H, S, s0, part.shape[2], D))

    # ---- TimeSelfAttention module --------------------------------------------------------
    def _tsa_params(self, x, wq, wk, wv, wo, B, S, H, head_width, scale, causal, time_major,
                    use_residual, use_layer_norm, gamma, beta, keep_mask, mode, biases=(None, None, None, None)):
        from ._lib import TsaParams
        E = x.shape[1]
        assert x.shape == (B * S, E) and x.dtype == torch.float32 and x.is_contiguous()
        HW = H * head_width
        assert wq.shape == (E, HW) and wk.shape == (E, HW) and wv.shape == (E, HW) and wo.shape == (HW, E)
        p = TsaParams()
        p.B, p.S, p.E, p.H, p.head_width = B, S, E, H, head_width
        p.causal, p.time_major = int(bool(causal)), int(bool(time_major))
        p.use_residual, p.use_layer_norm, p.mode = int(bool(use_residual)), int(bool(use_layer_norm)), int(mode)
        p.scale, p.score_clamp = float(scale), 0.0
        p.x = x.data_ptr()
        p.wq, p.wk, p.wv, p.wo = (w.data_ptr() for w in (wq, wk, wv, wo))
        if gamma is not None:
            p.ln_gamma, p.ln_beta = gamma.data_ptr(), beta.data_ptr()
        if keep_mask is not None:
            p.keep_mask = keep_mask.data_ptr()
        for name, b in zip(("bq", "bk", "bv", "bo"), biases):
            if b is not None:
                assert b.dtype == torch.float32 and b.is_contiguous()
                setattr(p, name, b.data_ptr())
        return p

    def _tsa_workspace(self, p, which):
        need = C.c_size_t(0)
        self.check(self.lib.ltca_tsa_workspace_bytes(C.byref(p), which, C.byref(need)))
        ws = self.workspace(need.value)
        p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
        return ws

    def tsa_saved_buffer(self, x, wq, wk, wv, wo, B, S, H, head_width, mode=_lib.MODE_AUTO, causal=False):
        """A buffer for the forward's intermediates: give it to ``tsa_fwd(saved=...)`` and then to
        ``tsa_bwd(saved=..., reuse_forward=True)`` to skip the backward's recomputation of the forward."""
        p = self._tsa_params(x, wq, wk, wv, wo, B, S, H, head_width, 1.0, causal, False, False, False, None, None,
                             None, mode, (None, None, None, None))
        need = C.c_size_t(0)
        self.check(self.lib.ltca_tsa_saved_bytes(C.byref(p), C.byref(need)))
        return torch.empty(need.value, dtype=torch.uint8, device=x.device)

    def tsa_weight_cache(self, x, wq, wk, wv, wo, B, S, H, head_width, mode=_lib.MODE_AUTO, causal=False):
        """A buffer for the reduced-precision copies of the weights (``ltca_tsa_params.weight_cache``): pass it as
        ``weight_cache=(buffer, False)`` to the first call and ``(buffer, True)`` while the weights stay unchanged."""
        p = self._tsa_params(x, wq, wk, wv, wo, B, S, H, head_width, 1.0, causal, False, False, False, None, None,
                             None, mode, (None, None, None, None))
        need = C.c_size_t(0)
        self.check(self.lib.ltca_tsa_weight_cache_bytes(C.byref(p), C.byref(need)))
        return torch.empty(max(need.value, 1), dtype=torch.uint8, device=x.device)

    @staticmethod
    def _attach_weight_cache(p, weight_cache):
        if weight_cache is not None:
            buf, valid = weight_cache
            p.weight_cache, p.weight_cache_bytes, p.weight_cache_valid = buf.data_ptr(), buf.numel(), int(valid)

    def tsa_fwd(self, x, wq, wk, wv, wo, B, S, H, head_width, scale=1.0, causal=False, time_major=True,
                use_residual=True, use_layer_norm=True, gamma=None, beta=None, keep_mask=None,
                mode=_lib.MODE_AUTO, bq=None, bk=None, bv=None, bo=None, saved=None, weight_cache=None):
        """out = LayerNorm(x + MHA(x)); x [B*S, E] fp32, weights as in ``ltca_tsa_params``."""
        p = self._tsa_params(x, wq, wk, wv, wo, B, S, H, head_width, scale, causal, time_major,
                             use_residual, use_layer_norm, gamma, beta, keep_mask, mode, (bq, bk, bv, bo))
        self._attach_weight_cache(p, weight_cache)
        if saved is not None:
            p.saved, p.saved_bytes = saved.data_ptr(), saved.numel()
        out = torch.empty_like(x)
        p.out = out.data_ptr()
        ws = self._tsa_workspace(p, 0)
        self.check(self.lib.ltca_tsa_fwd(self.handle, C.byref(p)))
        del ws
        return out

    def tsa_bwd(self, x, wq, wk, wv, wo, dy, B, S, H, head_width, scale=1.0, causal=False, time_major=True,
                keep_mask=None, mode=_lib.MODE_AUTO, bq=None, bk=None, bv=None, saved=None, reuse_forward=False,
                weight_cache=None):
        """(dx, dwq, dwk, dwv, dwo) of the module; LayerNorm and residual pass dy through."""
        p = self._tsa_params(x, wq, wk, wv, wo, B, S, H, head_width, scale, causal, time_major,
                             False, False, None, None, keep_mask, mode, (bq, bk, bv, None))
        self._attach_weight_cache(p, weight_cache)
        if saved is not None:
            p.saved, p.saved_bytes, p.reuse_forward = saved.data_ptr(), saved.numel(), int(reuse_forward)
        dx = torch.empty_like(x)
        # the four weight gradients are views of one allocation, so a multi-GPU caller sums them over the
        # ranks with a single collective on that allocation (shard.sum_weight_grads) without packing them
        flat = torch.empty(sum(w.numel() for w in (wq, wk, wv, wo)), dtype=wq.dtype, device=wq.device)
        dws, off = [], 0
        for w in (wq, wk, wv, wo):
            dws.append(flat[off:off + w.numel()].view(w.shape))
            off += w.numel()
        p.dy, p.dx = dy.data_ptr(), dx.data_ptr()
        p.dwq, p.dwk, p.dwv, p.dwo = (w.data_ptr() for w in dws)
        ws = self._tsa_workspace(p, 3)
        self.check(self.lib.ltca_tsa_bwd(self.handle, C.byref(p)))
        del ws
        return (dx, *dws)

    def fa_fwd(self, x, wq, wk, wv, wo, B, S, H, head_dim, biases=(None, None, None, None), gamma=None, beta=None,
               use_layer_norm=True, use_residual=True, keep_mask=None, dropout_prob=0.0, dropout_seed=0,
               score_clamp=10.0, mode=_lib.MODE_AUTO):
        """The reference's FlashAttention module: out = dropout(x + Wo MHA(LayerNorm(x)) + bo); x [B*S, E]
        batch-major rows, scale 1/sqrt(head_dim), score clamp 10."""
        p = self._tsa_params(x, wq, wk, wv, wo, B, S, H, head_dim, 1.0 / math.sqrt(head_dim), False, False,
                             use_residual, use_layer_norm, gamma, beta, keep_mask, mode, biases)
        p.pre_norm, p.score_clamp = 1, float(score_clamp)
        p.dropout_prob, p.dropout_seed = float(dropout_prob), int(dropout_seed)
        out = torch.empty_like(x)
        p.out = out.data_ptr()
        ws = self._tsa_workspace(p, 0)
        self.check(self.lib.ltca_tsa_fwd(self.handle, C.byref(p)))
        del ws
        return out

    def fa_bwd(self, x, wq, wk, wv, wo, dy, B, S, H, head_dim, biases=(None, None, None, None), gamma=None,
               beta=None, use_layer_norm=True, use_residual=True, keep_mask=None, dropout_prob=0.0,
               dropout_seed=0, score_clamp=10.0, mode=_lib.MODE_AUTO):
        """Backward of fa_fwd (an extension: the reference class has none).  Returns a dict with dx, dwq, dwk,
        dwv, dwo, dbq, dbk, dbv, dbo and, with LayerNorm, dgamma and dbeta."""
        p = self._tsa_params(x, wq, wk, wv, wo, B, S, H, head_dim, 1.0 / math.sqrt(head_dim), False, False,
                             use_residual, use_layer_norm, gamma, beta, keep_mask, mode, biases)
        p.pre_norm, p.score_clamp = 1, float(score_clamp)
        p.dropout_prob, p.dropout_seed = float(dropout_prob), int(dropout_seed)
        E, HW = x.shape[1], H * head_dim
        f32 = dict(dtype=torch.float32, device=x.device)
        g = dict(dx=torch.empty_like(x), dwq=torch.empty_like(wq), dwk=torch.empty_like(wk),
                 dwv=torch.empty_like(wv), dwo=torch.empty_like(wo), dbq=torch.empty(HW, **f32),
                 dbk=torch.empty(HW, **f32), dbv=torch.empty(HW, **f32), dbo=torch.empty(E, **f32))
        if use_layer_norm:
            g["dgamma"], g["dbeta"] = torch.empty(E, **f32), torch.empty(E, **f32)
        p.dy = dy.data_ptr()
        for name, t in g.items():
            setattr(p, name, t.data_ptr())
        ws = self._tsa_workspace(p, 3)
        self.check(self.lib.ltca_tsa_bwd(self.handle, C.byref(p)))
        del ws
        return g

    def uses_tensor_pipe(self, q, k, v, causal=False, mode=_lib.MODE_AUTO, backward=False) -> bool:
        o = q
        p = self._params(q, k, v, o, None, 1.0, causal, None, None, 0.0, mode)
        return bool(self.lib.ltca_attn_uses_tensor_pipe(C.byref(p), int(backward)))


_default: dict = {}


class HostStepPipeline:
    """Attention forward + backward steps whose operands live in pinned HOST memory and whose results
    return to pinned host memory, the way a caller that keeps its tensors on the host (the reference
    allocates and fills them there before every call) uses the library.

    Three streams - copy in, compute (the context's stream), copy out - and two sets of device buffers:
    while step i computes, the operands of step i+1 arrive and the results of step i-1 leave, so in
    steady state a step costs the slowest of the three stages instead of their sum (host-to-device and
    device-to-host traffic use the two directions of the link at the same time).
    """

    def __init__(self, ctx: "Context", compute_stream: torch.cuda.Stream, like_q: torch.Tensor,
                 like_k: torch.Tensor, causal: bool = True, deterministic: bool = False):
        self.ctx, self.causal, self.deterministic = ctx, causal, deterministic
        self.s_comp = compute_stream
        self.s_in, self.s_out = torch.cuda.Stream(like_q.device), torch.cuda.Stream(like_q.device)
        B, H, Sq, _ = like_q.shape
        mk = torch.empty_like
        self.bufs = []
        for _ in range(2):
            self.bufs.append(dict(q=mk(like_q), k=mk(like_k), v=mk(like_k), do=mk(like_q), o=mk(like_q),
                                  lse=torch.empty((B, H, Sq), dtype=torch.float32, device=like_q.device),
                                  dq=mk(like_q), dk=mk(like_k), dv=mk(like_k)))
        ev = lambda: [torch.cuda.Event() for _ in range(2)]
        self.ev_in, self.ev_comp, self.ev_out = ev(), ev(), ev()

    def run(self, host_in, host_out, steps: int, compute: bool = True):
        """`steps` forward+backward passes over host_in = (q, k, v, dout), results into
        host_out = (o, dq, dk, dv); all pinned host tensors.  Returns nothing; the caller synchronises.
        ``compute=False`` runs the same copies and the same stream dependencies without the kernels: what the
        host link alone allows."""
        hq, hk, hv, hdo = host_in
        ho, hdq, hdk, hdv = host_out
        for i in range(steps):
            j = i & 1
            b = self.bufs[j]
            with torch.cuda.stream(self.s_in):
                if i >= 2:
                    self.s_in.wait_event(self.ev_comp[j])        # step i-2 has read these operand buffers
                b["q"].copy_(hq, non_blocking=True); b["k"].copy_(hk, non_blocking=True)
                b["v"].copy_(hv, non_blocking=True); b["do"].copy_(hdo, non_blocking=True)
                self.ev_in[j].record(self.s_in)
            with torch.cuda.stream(self.s_comp):
                self.s_comp.wait_event(self.ev_in[j])
                if i >= 2:
                    self.s_comp.wait_event(self.ev_out[j])       # the results of step i-2 have left
                if compute:
                    self.ctx.attn_fwd(b["q"], b["k"], b["v"], causal=self.causal, mode=_lib.MODE_BF16,
                                      out=b["o"], lse=b["lse"])
                    self.ctx.attn_bwd(b["q"], b["k"], b["v"], b["o"], b["lse"], b["do"], causal=self.causal,
                                      mode=_lib.MODE_AUTO, dq=b["dq"], dk=b["dk"], dv=b["dv"],
                                      deterministic=self.deterministic)
                self.ev_comp[j].record(self.s_comp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_comp[j])
                ho.copy_(b["o"], non_blocking=True); hdq.copy_(b["dq"], non_blocking=True)
                hdk.copy_(b["dk"], non_blocking=True); hdv.copy_(b["dv"], non_blocking=True)
                self.ev_out[j].record(self.s_out)


def _ctx_for(t: torch.Tensor) -> Context:
    dev = t.device.index if t.device.index is not None else torch.cuda.current_device()
    if dev not in _default:
        _default[dev] = Context(dev)
    ctx = _default[dev]
    ctx.set_stream(torch.cuda.current_stream(dev))
    return ctx


def attention_forward(q, k, v, **kw):
    """O, lse = attention(q, k, v).  See :meth:`Context.attn_fwd`."""
    return _ctx_for(q).attn_fwd(q, k, v, **kw)


def attention_backward(q, k, v, o, lse, dout, **kw):
    """dq, dk, dv.  See :meth:`Context.attn_bwd`."""
    return _ctx_for(q).attn_bwd(q, k, v, o, lse, dout, **kw)


def attention_decode(q, k, v, kv_len=None, **kw):
    """Single-query step over a key/value cache.  See :meth:`Context.attn_decode`."""
    return _ctx_for(q).attn_decode(q, k, v, kv_len=kv_len, **kw)

"""TimeSelfAttention module against the reference's own cuDNN implementation.

tests/golden/ref_tsa_case*.npz were produced on a B200 by the reference's CuDNNTimeSelfAttention
(compiled from the reference sources, oracle/ref_tsa_driver.cu): input, output, input gradient
and the four projection matrices as the reference reads them out of cuDNN's weight buffer.  The
fp64 oracle is checked against them on CPU (this pins its layout, scale and ordering choices: rows
time-major, per-head projection width = input_dim, scale 1.0, no mask); the CUDA module is checked
against them through the C ABI on the GPU.  cuDNN's default math for fp32 data uses TF32 tensor
cores, so agreement is at the 1e-3 level, not fp32 round-off.
"""
import glob
import os

import numpy as np
import pytest

import oracle
from util import bf16_round, rel_l2

# Tensor-pipe MODULE bounds (derivation in tests/test_configs_gpu.py): every operand of a bf16 tensor-core product is
# rounded to bf16 (relative error up to 2^-8, RMS 1.6e-3), and the module chains three such stages, so against the
# oracle fed the bf16-rounded inputs the forward is held to rel-L2 5e-3 and max-abs 2^-7 x max(1, max|ref|), the
# gradients to rel-L2 7e-3 and the same max-abs.
MODULE_REL_L2, MODULE_GRAD_REL_L2, MODULE_MAX_ABS = 5e-3, 7e-3, 2.0 ** -7

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = sorted(glob.glob(os.path.join(HERE, "golden", "ref_tsa_case*.npz")))
TOL = 5e-3          # relative to the tensor's largest magnitude


def load(path):
    d = np.load(path)
    E, H, B, S = (int(d[k]) for k in ("E", "H", "B", "S"))
    # cuDNN hands out [heads, projected, input] views for Q/K/V and [heads, output, projected] for O;
    # the ABI wants y = x w with w [E, H*W] and ctx wo with wo [H*W, E]  (W = E here)
    qkv = [np.ascontiguousarray(np.transpose(d[n], (2, 0, 1)).reshape(E, H * E)) for n in ("wq", "wk", "wv")]
    wo = np.ascontiguousarray(np.transpose(d["wo"], (0, 2, 1)).reshape(H * E, E))
    return d, E, H, B, S, qkv, wo


def reference_weight_grads(d, E, H):
    """The reference's dWq, dWk, dWv, dWo (views of its gradient buffer with the weight buffer's descriptors,
    cuDNN_ops.cu:366-385 of the reference) in the ABI's matrix shapes, or None for a file without them."""
    if "dwq" not in d.files:
        return None
    g = [np.transpose(d[n], (2, 0, 1)).reshape(E, H * E) for n in ("dwq", "dwk", "dwv")]
    return g + [np.transpose(d["dwo"], (0, 2, 1)).reshape(H * E, E)]


def test_golden_files_exist():
    assert len(CASES) >= 4


@pytest.mark.parametrize("path", CASES)
def test_oracle_matches_reference_cudnn_module(path):
    d, E, H, B, S, (wq, wk, wv), wo = load(path)
    gamma, beta = np.ones(E, np.float32), np.zeros(E, np.float32)
    out, _ = oracle.tsa_fwd(d["x"], wq, wk, wv, wo, B, S, H, E, 1.0, False, True, bool(d["res"]), bool(d["ln"]),
                            gamma, beta)
    assert np.abs(out - d["y"]).max() < TOL * max(1.0, np.abs(d["y"]).max())
    if "dx" in d.files:
        grads = oracle.tsa_bwd(d["x"], wq, wk, wv, wo, d["dy"], B, S, H, E, 1.0, False, True)
        assert np.abs(grads[0] - d["dx"]).max() < TOL * max(1.0, np.abs(d["dx"]).max())
        ref_dw = reference_weight_grads(d, E, H)
        assert ref_dw is not None, "the golden files carry the reference's weight gradients"
        for name, g, r in zip(("dwq", "dwk", "dwv", "dwo"), grads[1:], ref_dw):
            assert np.abs(g - r).max() < TOL * max(1.0, np.abs(r).max()), name


@pytest.mark.gpu
@pytest.mark.parametrize("path", CASES)
def test_cuda_module_matches_reference_cudnn_module(ctx, path):
    import torch
    from cuda_ltc_b200 import _lib
    d, E, H, B, S, (wq, wk, wv), wo = load(path)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()
    x, dy, twq, twk, twv, two = (dev(a) for a in (d["x"], d["dy"], wq, wk, wv, wo))
    gamma, beta = torch.ones(E, device="cuda"), torch.zeros(E, device="cuda")
    out = ctx.tsa_fwd(x, twq, twk, twv, two, B, S, H, E, scale=1.0, time_major=True,
                      use_residual=bool(d["res"]), use_layer_norm=bool(d["ln"]), gamma=gamma, beta=beta,
                      mode=_lib.MODE_FP32)
    assert np.abs(out.cpu().numpy() - d["y"]).max() < TOL * max(1.0, np.abs(d["y"]).max())
    got = ctx.tsa_bwd(x, twq, twk, twv, two, dy, B, S, H, E, scale=1.0, time_major=True, mode=_lib.MODE_FP32)
    if "dx" in d.files:
        assert np.abs(got[0].cpu().numpy() - d["dx"]).max() < TOL * max(1.0, np.abs(d["dx"]).max())
        for name, g, r in zip(("dwq", "dwk", "dwv", "dwo"), got[1:], reference_weight_grads(d, E, H)):
            assert np.abs(g.cpu().numpy() - r).max() < TOL * max(1.0, np.abs(r).max()), name
    # and, tighter, against the fp64 oracle (same arithmetic, no TF32 in between)
    ref = oracle.tsa_bwd(d["x"], wq, wk, wv, wo, d["dy"], B, S, H, E, 1.0, False, True)
    for g, r in zip(got, ref):
        assert np.abs(g.cpu().numpy() - r).max() < 2e-4 * max(1.0, np.abs(r).max())


@pytest.mark.gpu
def test_cuda_module_compact_heads_causal(ctx):
    """The benchmark's form of the module (head width E/H, scale 1/sqrt(width), causal) on the
    tensor pipe, against the oracle."""
    import math
    import torch
    from cuda_ltc_b200 import _lib
    B, S, E, H = 2, 128, 256, 4
    W = E // H
    rng = np.random.default_rng(3)
    x = rng.standard_normal((B * S, E)).astype(np.float32)
    lim = math.sqrt(6.0 / (2 * E))
    wq, wk, wv = (rng.uniform(-lim, lim, (E, H * W)).astype(np.float32) for _ in range(3))
    wo = rng.uniform(-lim, lim, (H * W, E)).astype(np.float32)
    gamma, beta = np.ones(E, np.float32), np.zeros(E, np.float32)
    ref, _ = oracle.tsa_fwd(*(bf16_round(a) for a in (x, wq, wk, wv, wo)), B, S, H, W, 1 / math.sqrt(W), True, False,
                            True, True, gamma, beta)
    dev = lambda a: torch.from_numpy(a).cuda()
    out = ctx.tsa_fwd(dev(x), dev(wq), dev(wk), dev(wv), dev(wo), B, S, H, W, scale=1 / math.sqrt(W),
                      causal=True, time_major=False, gamma=dev(gamma), beta=dev(beta), mode=_lib.MODE_BF16)
    got = out.cpu().numpy()
    assert np.abs(got - ref).max() < MODULE_MAX_ABS * max(1.0, np.abs(ref).max())
    assert rel_l2(got, ref) < MODULE_REL_L2


TENSOR_MODULE_CASES = [
    # B, S, E, H, causal, time_major, biases
    (2, 128, 256, 4, True, False, False),
    (3, 100, 100, 2, False, True, True),      # E not a multiple of 8: padded bf16 rows; ragged tiles
    (8, 128, 256, 4, True, False, False),     # 1024 rows: the weight gradients split their contraction
]


@pytest.mark.gpu
@pytest.mark.parametrize("case", TENSOR_MODULE_CASES)
def test_cuda_module_tensor_pipe_forward_backward(ctx, case):
    """Every projection of the module on the tcgen05 GEMM (bf16 operands, fp32 accumulation), head
    width 64: forward output, input gradient and the four weight gradients against the oracle."""
    import math
    import torch
    from cuda_ltc_b200 import _lib
    B, S, E, H, causal, time_major, biases = case
    W = 64
    HW = H * W
    rng = np.random.default_rng(17)
    x = rng.standard_normal((B * S, E)).astype(np.float32)
    dy = rng.standard_normal((B * S, E)).astype(np.float32)
    lim = math.sqrt(6.0 / (E + HW))
    wq, wk, wv = (rng.uniform(-lim, lim, (E, HW)).astype(np.float32) for _ in range(3))
    wo = rng.uniform(-lim, lim, (HW, E)).astype(np.float32)
    bq, bk, bv = ((0.1 * rng.standard_normal(HW)).astype(np.float32) if biases else None for _ in range(3))
    bo = (0.1 * rng.standard_normal(E)).astype(np.float32) if biases else None
    gamma = (1.0 + 0.1 * rng.standard_normal(E)).astype(np.float32)
    beta = (0.1 * rng.standard_normal(E)).astype(np.float32)
    sc = 1 / math.sqrt(W)
    # the oracle consumes what the bf16 mode consumes: the module's inputs rounded to bf16 (biases stay fp32)
    xr, dyr, wqr, wkr, wvr, wor = (bf16_round(a) for a in (x, dy, wq, wk, wv, wo))
    ref, _ = oracle.tsa_fwd(xr, wqr, wkr, wvr, wor, B, S, H, W, sc, causal, time_major, True, True, gamma, beta,
                            bq, bk, bv, bo)
    gref = oracle.tsa_bwd(xr, wqr, wkr, wvr, wor, dyr, B, S, H, W, sc, causal, time_major, bq, bk, bv)
    dev = lambda a: None if a is None else torch.from_numpy(a).cuda()
    kw = dict(scale=sc, causal=causal, time_major=time_major, mode=_lib.MODE_BF16)
    out = ctx.tsa_fwd(dev(x), dev(wq), dev(wk), dev(wv), dev(wo), B, S, H, W, gamma=dev(gamma), beta=dev(beta),
                      bq=dev(bq), bk=dev(bk), bv=dev(bv), bo=dev(bo), **kw)
    got = ctx.tsa_bwd(dev(x), dev(wq), dev(wk), dev(wv), dev(wo), dev(dy), B, S, H, W,
                      bq=dev(bq), bk=dev(bk), bv=dev(bv), **kw)
    again = ctx.tsa_bwd(dev(x), dev(wq), dev(wk), dev(wv), dev(wo), dev(dy), B, S, H, W,
                        bq=dev(bq), bk=dev(bk), bv=dev(bv), **kw)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
    oh = out.cpu().numpy()
    assert np.abs(oh - ref).max() < MODULE_MAX_ABS * max(1.0, np.abs(ref).max())
    assert rel_l2(oh, ref) < MODULE_REL_L2
    for name, g, g2, r in zip(("dx", "dwq", "dwk", "dwv", "dwo"), got, again, gref):
        assert torch.equal(g, g2), f"{name}: two runs differ"
        gh = g.cpu().numpy().astype(np.float64)
        scale = max(1.0, float(np.abs(r).max()))
        assert np.abs(gh - r).max() < MODULE_MAX_ABS * scale, f"{name}: {np.abs(gh - r).max()} vs magnitude {scale}"
        assert rel_l2(gh, r) < MODULE_GRAD_REL_L2, f"{name}: rel-L2 {rel_l2(gh, r)}"


@pytest.mark.gpu
@pytest.mark.parametrize("mode_name", ["tensor", "exact"])
def test_backward_from_saved_forward_equals_backward_with_recomputation(ctx, mode_name):
    """A forward call that keeps its intermediates in a caller-held block, then a backward that reuses them:
    same bits as the default backward, which recomputes the forward; the forward output is unchanged too."""
    import math
    import torch
    from cuda_ltc_b200 import _lib
    from cuda_ltc_b200.api import LtcaError
    B, S, E, H, W = 4, 128, 256, 4, 64
    mode = _lib.MODE_BF16 if mode_name == "tensor" else _lib.MODE_FP32
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn((B * S, E), generator=g, device="cuda")
    dy = torch.randn((B * S, E), generator=g, device="cuda")
    lim = math.sqrt(6.0 / (2 * E))
    ws = [(torch.rand((E, H * W), generator=g, device="cuda") * 2 - 1) * lim for _ in range(3)]
    wo = (torch.rand((H * W, E), generator=g, device="cuda") * 2 - 1) * lim
    gamma, beta = torch.ones(E, device="cuda"), torch.zeros(E, device="cuda")
    kw = dict(scale=1 / math.sqrt(W), causal=True, time_major=False, mode=mode)
    plain_out = ctx.tsa_fwd(x, *ws, wo, B, S, H, W, gamma=gamma, beta=beta, **kw)
    plain = ctx.tsa_bwd(x, *ws, wo, dy, B, S, H, W, **kw)
    saved = ctx.tsa_saved_buffer(x, *ws, wo, B, S, H, W, mode=mode, causal=True)
    assert saved.numel() > 0
    out = ctx.tsa_fwd(x, *ws, wo, B, S, H, W, gamma=gamma, beta=beta, saved=saved, **kw)
    got = ctx.tsa_bwd(x, *ws, wo, dy, B, S, H, W, saved=saved, reuse_forward=True, **kw)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
    assert torch.equal(out, plain_out)
    for a, b in zip(got, plain):
        assert torch.equal(a, b)
    with pytest.raises(LtcaError):                       # a block that is too small is refused
        ctx.tsa_fwd(x, *ws, wo, B, S, H, W, gamma=gamma, beta=beta, saved=saved[:1024], **kw)


@pytest.mark.gpu
def test_cuda_module_reference_form_wide_heads(ctx):
    """The reference's largest configuration, (input_dim, heads) = (512, 8): every head is 512 wide
    (include/cuDNN_ops.h:166-169 of the reference), scale 1.0, no mask, time-major rows.  Forward and backward
    of the module against the oracle."""
    import torch
    from cuda_ltc_b200 import _lib
    B, S, E, H = 2, 12, 512, 8
    W = E
    rng = np.random.default_rng(23)
    x = (0.5 * rng.standard_normal((B * S, E))).astype(np.float32)
    dy = rng.standard_normal((B * S, E)).astype(np.float32)
    lim = np.sqrt(6.0 / (E + W))
    wq, wk, wv = (rng.uniform(-lim, lim, (E, H * W)).astype(np.float32) * 0.2 for _ in range(3))
    wo = rng.uniform(-lim, lim, (H * W, E)).astype(np.float32)
    gamma, beta = np.ones(E, np.float32), np.zeros(E, np.float32)
    ref, _ = oracle.tsa_fwd(x, wq, wk, wv, wo, B, S, H, W, 1.0, False, True, True, True, gamma, beta)
    gref = oracle.tsa_bwd(x, wq, wk, wv, wo, dy, B, S, H, W, 1.0, False, True)
    dev = lambda a: torch.from_numpy(a).cuda()
    kw = dict(scale=1.0, causal=False, time_major=True, mode=_lib.MODE_FP32)
    out = ctx.tsa_fwd(dev(x), dev(wq), dev(wk), dev(wv), dev(wo), B, S, H, W, gamma=dev(gamma), beta=dev(beta), **kw)
    got = ctx.tsa_bwd(dev(x), dev(wq), dev(wk), dev(wv), dev(wo), dev(dy), B, S, H, W, **kw)
    assert np.abs(out.cpu().numpy() - ref).max() < 1e-3
    for name, g, r in zip(("dx", "dwq", "dwk", "dwv", "dwo"), got, gref):
        assert np.abs(g.cpu().numpy() - r).max() < 1e-3 * max(1.0, np.abs(r).max()), name


WIDE_TENSOR_CASES = [
    # B, S, E, H, head width, scale, causal, time_major, mask, biases, mode
    (2, 12, 512, 8, 512, 1.0, False, True, False, False, "auto"),     # the reference's largest form: AUTO takes this path
    (4, 64, 256, 4, 256, 1.0, False, True, False, False, "auto"),
    (3, 40, 64, 2, 32, 32 ** -0.5, True, False, True, True, "bf16"),   # narrow heads on request, every mask kind
    (2, 100, 128, 2, 128, 1.0, True, True, False, False, "bf16"),     # width 128: streaming forward exists, backward does not
]


@pytest.mark.gpu
@pytest.mark.parametrize("case", WIDE_TENSOR_CASES)
def test_cuda_module_materialised_score_path(ctx, case):
    """Head widths the streaming kernels do not cover run on the tensor pipe through written-out score matrices
    (batched tcgen05 GEMMs).  x, Wq and Wk enter as two bf16 terms, so the scores are fp32-class even with the
    reference's scale of 1 and model-wide heads; v, P, ctx and Wo are single bf16 operands as in the compact
    module, hence the same bounds against the oracle fed the exact inputs."""
    import torch
    from cuda_ltc_b200 import _lib
    B, S, E, H, W, scale, causal, time_major, use_mask, biases, mode_name = case
    mode = _lib.MODE_AUTO if mode_name == "auto" else _lib.MODE_BF16
    HW = H * W
    rng = np.random.default_rng(31)
    x = (0.5 * rng.standard_normal((B * S, E))).astype(np.float32)
    dy = rng.standard_normal((B * S, E)).astype(np.float32)
    lim = np.sqrt(6.0 / (E + W))
    amp = 0.25 if W > 128 else 1.0                 # keeps the unscaled scores of model-wide heads at magnitude ~10
    wq, wk = (rng.uniform(-lim, lim, (E, HW)).astype(np.float32) * amp for _ in range(2))
    wv = rng.uniform(-lim, lim, (E, HW)).astype(np.float32)
    wo = rng.uniform(-lim, lim, (HW, E)).astype(np.float32)
    bq, bk, bv = ((0.1 * rng.standard_normal(HW)).astype(np.float32) if biases else None for _ in range(3))
    gamma, beta = np.ones(E, np.float32), np.zeros(E, np.float32)
    m = None
    if use_mask:
        m = (rng.random((B, S, S)) < 0.8).astype(np.float32)
        m[:, np.arange(S), np.arange(S)] = 1.0
    ref, y_ref = oracle.tsa_fwd(x, wq, wk, wv, wo, B, S, H, W, scale, causal, time_major, True, True, gamma, beta,
                                bq, bk, bv, None, m)
    gref = oracle.tsa_bwd(x, wq, wk, wv, wo, dy, B, S, H, W, scale, causal, time_major, bq, bk, bv, m)
    dev = lambda a: None if a is None else torch.from_numpy(a).cuda()
    kw = dict(scale=scale, causal=causal, time_major=time_major, mode=mode, keep_mask=dev(m))
    args = (dev(x), dev(wq), dev(wk), dev(wv), dev(wo))
    y = ctx.tsa_fwd(*args, B, S, H, W, use_residual=False, use_layer_norm=False, bq=dev(bq), bk=dev(bk), bv=dev(bv), **kw)
    out = ctx.tsa_fwd(*args, B, S, H, W, gamma=dev(gamma), beta=dev(beta), bq=dev(bq), bk=dev(bk), bv=dev(bv), **kw)
    got = ctx.tsa_bwd(*args, dev(dy), B, S, H, W, bq=dev(bq), bk=dev(bk), bv=dev(bv), **kw)
    again = ctx.tsa_bwd(*args, dev(dy), B, S, H, W, bq=dev(bq), bk=dev(bk), bv=dev(bv), **kw)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
    for name, g, r in (("y", y, y_ref), ("out", out, ref)):
        gh = g.cpu().numpy()
        assert rel_l2(gh, r) < MODULE_REL_L2, f"{name}: rel-L2 {rel_l2(gh, r)}"
        assert np.abs(gh - r).max() < MODULE_MAX_ABS * max(1.0, np.abs(r).max()), name
    for name, g, g2, r in zip(("dx", "dwq", "dwk", "dwv", "dwo"), got, again, gref):
        assert torch.equal(g, g2), f"{name}: two runs differ"
        gh = g.cpu().numpy().astype(np.float64)
        assert rel_l2(gh, r) < MODULE_GRAD_REL_L2, f"{name}: rel-L2 {rel_l2(gh, r)}"
        assert np.abs(gh - r).max() < MODULE_MAX_ABS * max(1.0, np.abs(r).max()), name
    # A forward that keeps its intermediates, then two backward calls from the same block (the reference's
    # caller runs backwardWeights and then backward after one forward): both equal the recomputing call,
    # so the first one left the kept probabilities as it found them.
    saved = ctx.tsa_saved_buffer(*args, B, S, H, W, mode=mode, causal=causal)
    out_kept = ctx.tsa_fwd(*args, B, S, H, W, gamma=dev(gamma), beta=dev(beta), bq=dev(bq), bk=dev(bk), bv=dev(bv),
                           saved=saved, **kw)
    assert torch.equal(out_kept, out)
    for _ in range(2):
        kept = ctx.tsa_bwd(*args, dev(dy), B, S, H, W, bq=dev(bq), bk=dev(bk), bv=dev(bv), saved=saved,
                           reuse_forward=True, **kw)
        for name, g, g2 in zip(("dx", "dwq", "dwk", "dwv", "dwo"), got, kept):
            assert torch.equal(g, g2), f"{name}: kept forward differs from the recomputed one"
    torch.cuda.synchronize()
    assert ctx.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("form", ["compact", "reference"])
def test_kept_weight_copies_give_the_same_bits(ctx, form):
    """``weight_cache``: the first call writes the weights' reduced-precision copies into the caller's block, later
    calls run from them; outputs and gradients equal the converting calls bit for bit.  When the weights change and
    the caller clears the flag, the block follows; if the caller leaves it set, the stale copies are what is used
    (that is the contract)."""
    import torch
    from cuda_ltc_b200 import _lib
    from cuda_ltc_b200.api import LtcaError
    if form == "compact":
        B, S, E, H, W, kw = 4, 64, 128, 2, 64, dict(scale=0.125, causal=True, time_major=False, mode=_lib.MODE_BF16)
    else:
        B, S, E, H, W, kw = 2, 24, 256, 2, 256, dict(scale=1.0, causal=False, time_major=True, mode=_lib.MODE_AUTO)
    g = torch.Generator(device="cuda").manual_seed(5)
    rnd = lambda *shape: torch.randn(shape, generator=g, device="cuda")
    x, dy = 0.5 * rnd(B * S, E), rnd(B * S, E)
    ws = [0.05 * rnd(E, H * W) for _ in range(3)]
    wo = 0.05 * rnd(H * W, E)
    gamma, beta = torch.ones(E, device="cuda"), torch.zeros(E, device="cuda")
    plain_out = ctx.tsa_fwd(x, *ws, wo, B, S, H, W, gamma=gamma, beta=beta, **kw)
    plain = ctx.tsa_bwd(x, *ws, wo, dy, B, S, H, W, **kw)
    cache = ctx.tsa_weight_cache(x, *ws, wo, B, S, H, W, mode=kw["mode"], causal=kw["causal"])
    assert cache.numel() > 1
    for valid in (False, True, True):
        out = ctx.tsa_fwd(x, *ws, wo, B, S, H, W, gamma=gamma, beta=beta, weight_cache=(cache, valid), **kw)
        got = ctx.tsa_bwd(x, *ws, wo, dy, B, S, H, W, weight_cache=(cache, True), **kw)
        assert torch.equal(out, plain_out)
        for a, b in zip(got, plain):
            assert torch.equal(a, b)
    ws2 = [w * 1.5 for w in ws]
    new_out = ctx.tsa_fwd(x, *ws2, wo, B, S, H, W, gamma=gamma, beta=beta, **kw)
    stale = ctx.tsa_fwd(x, *ws2, wo, B, S, H, W, gamma=gamma, beta=beta, weight_cache=(cache, True), **kw)
    fresh = ctx.tsa_fwd(x, *ws2, wo, B, S, H, W, gamma=gamma, beta=beta, weight_cache=(cache, False), **kw)
    assert torch.equal(stale, plain_out) and torch.equal(fresh, new_out) and not torch.equal(new_out, plain_out)
    with pytest.raises(LtcaError):                       # a block that is too small is refused
        ctx.tsa_fwd(x, *ws, wo, B, S, H, W, gamma=gamma, beta=beta, weight_cache=(cache[:256], False), **kw)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("path", [c for c in CASES if int(np.load(c)["E"]) % 8 == 0])
def test_materialised_score_path_matches_reference_cudnn_module(ctx, path):
    """The same path against the reference's own cuDNN module (golden vectors), at the 2e-2 of the largest
    magnitude that separates two reduced-precision evaluations of the reference's unscaled attention."""
    import torch
    from cuda_ltc_b200 import _lib
    d, E, H, B, S, (wq, wk, wv), wo = load(path)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()
    x, dy, twq, twk, twv, two = (dev(a) for a in (d["x"], d["dy"], wq, wk, wv, wo))
    gamma, beta = torch.ones(E, device="cuda"), torch.zeros(E, device="cuda")
    kw = dict(scale=1.0, time_major=True, mode=_lib.MODE_BF16)
    out = ctx.tsa_fwd(x, twq, twk, twv, two, B, S, H, E, use_residual=bool(d["res"]), use_layer_norm=bool(d["ln"]),
                      gamma=gamma, beta=beta, **kw)
    got = ctx.tsa_bwd(x, twq, twk, twv, two, dy, B, S, H, E, **kw)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
    tol = 2e-2
    assert np.abs(out.cpu().numpy() - d["y"]).max() < tol * max(1.0, np.abs(d["y"]).max())
    assert np.abs(got[0].cpu().numpy() - d["dx"]).max() < tol * max(1.0, np.abs(d["dx"]).max())
    for name, g, r in zip(("dwq", "dwk", "dwv", "dwo"), got[1:], reference_weight_grads(d, E, H)):
        assert np.abs(g.cpu().numpy() - r).max() < tol * max(1.0, np.abs(r).max()), name

"""The C++ binding (include/ltc_attn_shim.hpp) executed on the GPU.

oracle/_ref/shim_driver is built from oracle/shim_driver.cu against the reference's own headers and objects
and against libltc_attn.so (oracle/Makefile; it needs the reference checkout, so it is built in advance and
only run here).  Its `check` command reproduces the properties the reference's tests pin for the class and
the drop-in checks against the reference's cuDNN module in the same process; this test asserts on its
verdict lines and then compares the weight files the classes wrote with the reference's initialisation
recipes evaluated in numpy.
"""
import os
import struct
import subprocess

import numpy as np
import pytest

from util import reference_tsa_weight_blob, std_uniform_stream

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DRIVER = os.path.join(ROOT, "oracle", "_ref", "shim_driver")

REQUIRED = [
    "ctor_rejects_indivisible", "ctor_rejects_zero_heads", "ctor_rejects_negative_dim", "getters",
    "deterministic_two_instances", "save_load_same_output", "load_refuses_other_shape", "shape_sweep",
    "backward_repeatable_e8", "backward_repeatable_e6", "training_step_call_order", "mask_ignored_by_default",
    "mask_honoured_on_request", "binding_equals_direct_call", "device_status_clean",
    "fa_forward_shape_finite", "fa_deterministic_two_instances", "fa_save_load_same_output", "fa_backward",
    "no_cuda_error",
]
WITH_REFERENCE = [
    "same_seed_weight_file_is_byte_identical", "forward_vs_reference_module", "backward_vs_reference_module",
    "reference_weight_file_loads", "reference_loads_binding_file",
]


@pytest.fixture(scope="module")
def run(tmp_path_factory):
    if not os.path.exists(DRIVER):
        pytest.skip("oracle/_ref/shim_driver has not been built (it needs the reference checkout)")
    out = tmp_path_factory.mktemp("shim")
    r = subprocess.run([DRIVER, "check", str(out)], capture_output=True, text=True, timeout=600)
    checks = {}
    for line in r.stdout.splitlines():
        t = line.split()
        if len(t) == 5 and t[0] == "CHECK":
            checks[t[1]] = (float(t[2]), float(t[3]), t[4])
    return r, checks, str(out)


def test_binding_passes_the_reference_class_properties(run):
    r, checks, _ = run
    failed = {k: v for k, v in checks.items() if v[2] != "PASS"}
    assert r.returncode == 0 and not failed, f"{failed}\n{r.stdout[-3000:]}\n{r.stderr[-2000:]}"
    for name in REQUIRED:
        assert name in checks, f"{name} did not run\n{r.stdout[-3000:]}"
    if "NOTE reference cuDNN module unavailable" not in r.stdout:
        for name in WITH_REFERENCE:
            assert name in checks, f"{name} did not run"


def test_time_self_attention_file_follows_the_reference_recipe(run):
    _, _, out = run
    raw = open(os.path.join(out, "shim_tsa_weights.bin"), "rb").read()
    magic, version, nbytes = struct.unpack("<IIQ", raw[:16])
    assert (magic, version, nbytes) == (0x43444E4E, 1, len(raw) - 16)
    assert np.array_equal(np.frombuffer(raw[16:], dtype=np.float32), reference_tsa_weight_blob(64, 2, 12345))
    ln = np.fromfile(os.path.join(out, "shim_tsa_weights.bin.layernorm"), dtype=np.float32)
    assert np.array_equal(ln, np.concatenate([np.ones(64, np.float32), np.zeros(64, np.float32)]))


def test_flash_attention_file_follows_the_reference_recipe(run):
    """Header and payload of FlashAttention::saveWeights (reference src/ml/flash_attention.cu:619-687) with the
    weights of FlashAttention::initializeWeights (:551-611): (Wq[i], Wk[i], Wv[i]) interleaved, then Wo."""
    _, _, out = run
    raw = open(os.path.join(out, "shim_fa_weights.bin"), "rb").read()
    E, D, H = 32, 16, 2
    M = D * H
    in_dim, head_dim, heads, model_dim, drop, ln, res = struct.unpack("<iiiif??", raw[:22])
    assert (in_dim, head_dim, heads, model_dim, drop, ln, res) == (E, D, H, M, 0.0, True, True)
    body = np.frombuffer(raw[22:], dtype=np.float32)
    lim = np.sqrt(np.float32(6.0) / np.float32(E + M))
    stream = std_uniform_stream(12345, 4 * E * M, -lim, lim)
    qkv = stream[:3 * E * M].reshape(E * M, 3)
    want = np.concatenate([qkv[:, 0], qkv[:, 1], qkv[:, 2], stream[3 * E * M:], np.zeros(3 * M + E, np.float32),
                           np.ones(E, np.float32), np.zeros(E, np.float32)])
    assert body.size == want.size and np.array_equal(body, want)

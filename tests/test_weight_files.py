"""Weight files of the TimeSelfAttention module: layout and seeded initialisation, on CPU.

tests/golden/ref_tsa_weights_case{0,1}.bin are files the reference's own cuDNN module wrote with its
saveWeights on a B200 (tests/golden/make_tsa_golden.py keeps them beside the vectors).  Two facts are
pinned here because the C++ binding (include/ltc_attn_shim.hpp) relies on them:

* payload order: header (u32 0x43444E4E, u32 1, u64 byte count, reference src/ml/cuDNN_ops.cu:391-420), then
  Wq, Wk, Wv as row-major [E, H*E] and Wo as row-major [H*E, E] -- the matrices of the C ABI
  (``ltca_tsa_params``), so a reference file loads into the binding without any permutation;
* initialisation: one mt19937(seed), matrices drawn in the order Q, K, V, O in memory order with limit
  sqrt(6 / (E + E)) (reference src/ml/cuDNN_ops.cu:34-96), so equal seeds give byte-identical files.
"""
import os
import struct

import numpy as np
import pytest

from util import reference_tsa_weight_blob

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = [(0, 8, 2, 42), (1, 6, 2, 43)]          # golden case, input_dim, heads, seed (oracle/ref_tsa_driver.cu)


def read_blob(path):
    raw = open(path, "rb").read()
    magic, version, nbytes = struct.unpack("<IIQ", raw[:16])
    assert magic == 0x43444E4E and version == 1 and nbytes == len(raw) - 16
    return np.frombuffer(raw[16:], dtype=np.float32)


@pytest.mark.parametrize("case", CASES)
def test_reference_weight_file_is_the_abi_layout(case):
    idx, E, H, _ = case
    blob = read_blob(os.path.join(HERE, "golden", f"ref_tsa_weights_case{idx}.bin"))
    d = np.load(os.path.join(HERE, "golden", f"ref_tsa_case{idx}.npz"))
    n = E * H * E
    assert blob.size == 4 * n
    for i, name in enumerate(("wq", "wk", "wv")):
        w_abi = blob[i * n:(i + 1) * n].reshape(E, H * E)            # y = x w
        # cuDNN's own description of the same bytes: [heads, projected, input]
        assert np.array_equal(w_abi, np.transpose(d[name], (2, 0, 1)).reshape(E, H * E))
    wo_abi = blob[3 * n:].reshape(H * E, E)
    assert np.array_equal(wo_abi, np.transpose(d["wo"], (0, 2, 1)).reshape(H * E, E))


@pytest.mark.parametrize("case", CASES)
def test_seeded_initialisation_reproduces_the_reference_file(case):
    idx, E, H, seed = case
    blob = read_blob(os.path.join(HERE, "golden", f"ref_tsa_weights_case{idx}.bin"))
    assert np.array_equal(blob, reference_tsa_weight_blob(E, H, seed))

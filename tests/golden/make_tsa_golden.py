"""Turns the dump of oracle/_ref/ref_tsa_driver (the reference's own cuDNN TimeSelfAttention,
run on a B200) into the committed golden vectors tests/golden/ref_tsa_case*.npz.

    ./oracle/_ref/ref_tsa_driver dump <dir>         # on a GPU machine
    python tests/golden/make_tsa_golden.py <dir>

The projection matrices are stored as the reference reads them (cudnnGetMultiHeadAttnWeights,
reference src/ml/cuDNN_ops.cu:54-70): a [heads, a, b] view with explicit strides; the arrays
saved here are dense [heads, a, b] copies of that view, and `<name>_offset` is the byte offset of
the view inside the weight buffer.  The weight gradients (dwq ... dwo, where the driver could read
them) are the same views of the reference's gradient buffer.  For the two smallest cases the
module's own weight file, exactly as the reference's saveWeights wrote it, is kept beside the
vectors as ref_tsa_weights_case<i>.bin.
"""
import os
import shutil
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main(src):
    lines = open(os.path.join(src, "manifest.txt")).read().splitlines()
    i = 0
    while i < len(lines):
        t = lines[i].split()
        if t[0] != "case" or t[2] == "failed:":
            i += 1
            continue
        idx = int(t[1])
        meta = {t[j]: int(t[j + 1]) for j in range(2, len(t) - 1, 2)}
        out = {k: np.int64(v) for k, v in meta.items() if k in ("E", "H", "B", "S", "ln", "res")}
        for name in ("wq", "wk", "wv", "wo"):
            i += 1
            w = lines[i].split()
            assert w[0] == name
            nd = int(w[2])
            dims = [int(x) for x in w[4:4 + nd]]
            strides = [int(x) for x in w[5 + nd:5 + 2 * nd]]
            raw = np.fromfile(os.path.join(src, f"{name}{idx}.f32"), dtype=np.float32)
            dense = np.lib.stride_tricks.as_strided(raw, shape=dims, strides=[4 * s for s in strides]).copy()
            out[name] = dense
            out[name + "_strides"] = np.array(strides, dtype=np.int64)
            offset = int(w[w.index("offset") + 1])
            out[name + "_offset"] = np.int64(offset)
            if meta.get("dw"):
                graw = np.fromfile(os.path.join(src, f"dw{idx}.bin"), dtype=np.float32)[offset // 4:]
                out["d" + name] = np.lib.stride_tricks.as_strided(
                    graw, shape=dims, strides=[4 * s for s in strides]).copy()
        n = (meta["B"] * meta["S"], meta["E"])
        for name in ("x", "dy", "y") + (("dx",) if meta["dx"] else ()):
            out[name] = np.fromfile(os.path.join(src, f"{name}{idx}.f32"), dtype=np.float32).reshape(n)
        np.savez_compressed(os.path.join(HERE, f"ref_tsa_case{idx}.npz"), **out)
        if meta["blob"] <= 4096:
            shutil.copyfile(os.path.join(src, f"w{idx}.bin"), os.path.join(HERE, f"ref_tsa_weights_case{idx}.bin"))
        print("wrote case", idx, {k: v for k, v in meta.items()})
        i += 1


if __name__ == "__main__":
    main(sys.argv[1])

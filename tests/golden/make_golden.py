"""Generates tests/golden/ref_flash_case*.npz from the reference's own kernel.

Needs a GPU: runs ``oracle/_ref/ref_driver flash`` (the reference's flashAttentionKernel, built
unmodified from the reference checkout by oracle/Makefile) and packs its raw dumps.

    python tests/golden/make_golden.py [output_dir]     # default: tests/golden
"""
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def main(out_dir: str) -> None:
    driver = os.path.join(ROOT, "oracle", "_ref", "ref_driver")
    os.makedirs(out_dir, exist_ok=True)
    with tempfile.TemporaryDirectory() as tmp:
        subprocess.check_call([driver, "flash", tmp])
        for line in open(os.path.join(tmp, "manifest.txt")):
            idx, B, H, S, D, mask_kind, scale, clamp = line.split()
            B, H, S, D = int(B), int(H), int(S), int(D)
            load = lambda n, shape: np.fromfile(os.path.join(tmp, f"case{idx}_{n}.bin"), dtype=np.float32).reshape(shape)
            arrays = dict(q=load("q", (B, H, S, D)), k=load("k", (B, H, S, D)), v=load("v", (B, H, S, D)),
                          out=load("out", (B, H, S, D)), scale=np.float32(scale), clamp=np.float32(clamp))
            if int(mask_kind):
                arrays["mask"] = load("mask", (B, S, S))
            np.savez_compressed(os.path.join(out_dir, f"ref_flash_case{idx}.npz"), **arrays)
            print("wrote case", idx, (B, H, S, D), "mask" if int(mask_kind) else "")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else HERE)

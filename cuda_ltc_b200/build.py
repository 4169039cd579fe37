"""Builds libltc_attn.so (the C-ABI library) in-tree with nvcc for sm_100a.

Run as ``python -m cuda_ltc_b200.build`` or call :func:`build_library`.  Objects go to
``cuda_ltc_b200/build/`` and the library to ``cuda_ltc_b200/libltc_attn.so``; a source file is
recompiled only when it or one of the headers is newer than its object.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libltc_attn.so")
OBJ_DIR = os.path.join(HERE, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers_mtime():
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    paths.append(os.path.join(HERE, "..", "include", "ltc_attn.h"))
    return max(os.path.getmtime(p) for p in paths)


def _compile(src: str, obj: str) -> str:
    cmd = ["nvcc", *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    log = r.stdout + r.stderr
    with open(obj + ".log", "w") as f:
        f.write(" ".join(cmd) + "\n" + log)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{log}")
    return log


def build_library(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdr_m = _headers_mtime()
    todo, objs = [], []
    for src in _sources():
        obj = os.path.join(OBJ_DIR, src[:-3] + ".o")
        objs.append(obj)
        sm = max(os.path.getmtime(os.path.join(CSRC, src)), hdr_m)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < sm:
            todo.append((src, obj))
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            for log in ex.map(lambda so: _compile(*so), todo):
                if verbose:
                    print(log)
    if todo or not os.path.exists(OUT):
        cmd = ["nvcc", "-shared", "-o", OUT, *objs, "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    return OUT


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))

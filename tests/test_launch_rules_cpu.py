"""Source-level rule for the dependent launches: a kernel that is launched with programmatic stream serialisation
(`launch_dependent`, `launch_dependent_if`) may start while the kernel before it still runs, so its body must contain
the wait that holds it back before the first access to global memory (`grid_dependency_wait`).  No GPU needed."""
import os
import re

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "cuda_ltc_b200", "csrc")


def _sources():
    out = {}
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".cu", ".cuh", ".h")):
            with open(os.path.join(CSRC, name)) as f:
                out[name] = f.read()
    return out


def _kernel_bodies(text):
    """name -> body for every __global__ function of a source file (brace matching)."""
    bodies = {}
    for m in re.finditer(r"__global__\s+void(?:\s+__launch_bounds__\([^)]*\))?\s+(\w+)\s*\(", text):
        i = text.index("{", m.end())
        depth, j = 1, i + 1
        while depth:
            depth += {"{": 1, "}": -1}.get(text[j], 0)
            j += 1
        bodies[m.group(1)] = text[i:j]
    return bodies


def test_every_dependent_launch_targets_a_kernel_that_waits():
    src = _sources()
    bodies = {}
    for text in src.values():
        bodies.update(_kernel_bodies(text))
    launched = set()
    for name, text in src.items():
        for m in re.finditer(r"launch_dependent(?:_if)?\(\s*([^;]*?);", text, flags=re.S):
            args = m.group(1)
            if args.startswith(("bool dependent", "void (*kern)", "true, kern")):
                continue                                    # the helpers' own definitions
            first = args.split(",")[1] if "launch_dependent_if" in m.group(0) else args.split(",")[0]
            launched.add(first.strip())
    assert launched, "no dependent launch found: the pattern of this test is out of date"
    # local aliases of kernels (function pointers picked at run time) and the kernels they stand for
    alias = {
        "kern": None,                                        # resolved below, per file
        "kdq": "attn_bwd_dq_sm100_kernel", "kdkv": "attn_bwd_dkv_sm100_kernel",
        "fwd_kernel": "wide_softmax_fwd_rows_kernel", "bwd_kernel": "wide_softmax_bwd_rows_kernel",
    }
    names = set()
    for k in launched:
        base = re.sub(r"<.*", "", k)
        if base == "kern":
            names.update({"gemm_bf16_sm100_kernel", "attn_fwd_sm100_kernel"})
        elif base in alias:
            names.add(alias[base])
            if base == "fwd_kernel":
                names.add("wide_softmax_fwd_kernel")
            if base == "bwd_kernel":
                names.add("wide_softmax_bwd_kernel")
        else:
            names.add(base)
    for k in sorted(names):
        assert k in bodies, f"{k}: launched as a dependent kernel but not found"
        assert "grid_dependency_wait()" in bodies[k], f"{k} is launched as a dependent kernel but never waits"


def test_waiting_kernels_touch_no_kernel_argument_memory_before_the_wait():
    """Before its wait a kernel may set up shared memory, barriers and tensor memory only: no pointer of the argument
    block is dereferenced there (the key lengths get a wait of their own where they are read early)."""
    for text in _sources().values():
        for name, body in _kernel_bodies(text).items():
            k = body.find("grid_dependency_wait()")
            if k < 0:
                continue
            before = body[:k]
            assert not re.search(r"\ba\.\w+\[|\bg\.\w+\[[^\]]*\]\s*[^;=]*;|__ldg\(|atomic\w+\(", before), name

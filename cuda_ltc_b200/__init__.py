"""B200 (sm_100a) attention path for the CUDA_LTC model family.

``cuda_ltc_b200`` holds the CUDA kernels and the C-ABI library (``csrc/``), its ctypes binding
(``_lib``) and a thin torch-tensor front end (``api``) used by the tests and the benchmark.
"""
from . import _lib  # noqa: F401
from .api import (  # noqa: F401
    Context,
    HostStepPipeline,
    LtcaError,
    attention_backward,
    attention_decode,
    attention_forward,
)

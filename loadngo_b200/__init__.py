"""cuda-compute for loadngo's gpt-oss attention path on NVIDIA B200 (sm_100a).

The product is `libcuda_compute.so` (C ABI in include/cuda_compute.h).  This package holds its
sources (`csrc/`), a ctypes mirror of the reference's `metal-compute` interface (`compute`) and
the host-side page bookkeeping (`paged`).  Nothing here computes attention on the CPU.
"""
from . import compute, paged  # noqa: F401

__all__ = ["compute", "paged"]

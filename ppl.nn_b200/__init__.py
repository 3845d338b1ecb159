"""B200 (sm_100a) kernels for ppl.nn's INT8-KV cache attention path.

Layout:
  csrc/      CUDA kernels and the extern "C" layer (include/ppl_nn_b200.h)
  host/      C++ mirror of the llm_cuda operator/kernel classes that call the C ABI
  capi.py    ctypes binding of the C ABI
  ops.py     operator-level face on torch tensors (tests, benchmark)
  workloads.py  seeded synthetic workloads of the benchmark configurations
  build.py   nvcc recipe
"""
from . import capi  # noqa: F401

__all__ = ["capi"]

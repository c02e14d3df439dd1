"""cuda-llm_b200: the memory-bound tensor operators of cuda-llm, rebuilt for B200 (sm_100a).

Layout
  csrc/         CUDA kernels and the C ABI (include/b2ops.h at the repository root)
  csrc/llm/     C++ functions with the reference's own signatures (include/llm/*.h)
  lib.py        ctypes binding of the C ABI (no fallback: a missing library is an error)
  ops.py        the reference's operator names over torch tensors
  sharded.py    row sharding and the vocabulary-sharded argmax / softmax exchange
  workloads.py  seeded synthetic inputs of the benchmark configurations
  build.py      in-tree nvcc build
"""
from . import workloads  # numpy only

__all__ = ["workloads", "lib", "ops", "sharded", "hostio", "build"]


def __getattr__(name):
    # torch- and ctypes-backed modules load on first use so that `import cuda_llm_b200`
    # stays cheap; they raise if the CUDA library has not been built.
    if name in ("lib", "ops", "sharded", "hostio", "build"):
        import importlib
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)

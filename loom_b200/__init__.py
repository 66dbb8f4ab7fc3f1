"""loom_b200 -- B200 (sm_100a) implementation of Loom's BitNet ternary x int8 linear path.

The product is the CUDA shared library `lib/libloom_b200.so` behind the C ABI of
`include/loom_b200.h`.  This package holds its sources (`csrc/`), the build recipe and a thin
ctypes binding used by the tests and the benchmark.  There is no CPU fallback anywhere in it.
"""
from .cabi import Context, LoomB200Error, Weight, lib, lib_path  # noqa: F401

__all__ = ["Context", "Weight", "LoomB200Error", "lib", "lib_path"]

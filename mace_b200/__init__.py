"""mace_b200 -- B200-native device library for MACE's quantized-GEMM / conv path.

The product is the C-ABI shared library ``libmace_b200.so`` (declared in
``include/mace_b200.h``) and the C++ host layer under ``mace_b200/host``.  This
Python package is only a loader used by the tests and the benchmark: it binds
the C ABI with ctypes and fails loudly when the library has not been built.
There is no CPU fallback.
"""
from .capi import Context, MaceB200Error, lib, lib_path, build  # noqa: F401

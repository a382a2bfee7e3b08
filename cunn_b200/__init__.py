"""cunn_b200 — B200 (sm_100a) kernels for the THCUNN convolutional hot path.

The product is the shared library ``cunn_b200/lib/libTHCUNN.so`` (CUDA kernels
behind a C ABI).  This package is the Python host side used by the tests and
the benchmark: ``functional`` calls the flat ABI on torch CUDA tensors (torch
only provides device memory and streams), ``thnn`` drives the ``THNN_Cuda*``
entry points the way the reference's LuaJIT FFI binding does.
"""
from . import _lib  # noqa: F401  (raises if the library is not built)
from ._lib import CunnError, SO_PATH, device_status  # noqa: F401

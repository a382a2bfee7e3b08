"""cunn_b200 — B200 (sm_100a) kernels for the THCUNN convolutional hot path.

The product is the shared library ``cunn_b200/lib/libTHCUNN.so`` (CUDA kernels
behind a C ABI).  This package is the Python host side used by the tests and
the benchmark: ``functional`` calls the flat ABI on torch CUDA tensors (torch
only provides device memory and streams), ``thnn`` drives the ``THNN_Cuda*``
entry points the way the reference's LuaJIT FFI binding does.

The library is loaded on first use (``cunn_b200._lib``); if it has not been
built that import raises — there is no CPU or PyTorch fallback.  ``python -m
cunn_b200.build`` builds it.
"""


def __getattr__(name):
    if name in ("CunnError", "SO_PATH", "device_status", "lib"):
        from . import _lib
        return getattr(_lib, name)
    raise AttributeError(name)

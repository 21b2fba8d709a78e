"""cactus_b200: B200 (sm_100a) kernels for the quantised mul_mat + flash-attention path of cactus's ggml runtime.

The product is ``lib/libcactus_b200.so`` (C ABI in ``include/cactus_b200.h``) and the ggml backend
plug-in built on it; this package is the Python host-side mirror used by tests and the benchmark.
"""
from ._lib import B200Error, LIB_PATH, lib  # noqa: F401

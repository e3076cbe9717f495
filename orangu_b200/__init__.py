"""B200-native (sm_100a) backend for orangu-server's quantized decode path.

The product is the shared library ``_lib/liborangu_b200.so`` (CUDA kernels behind the C ABI of
``include/orangu_b200.h``).  This package is the host-side mirror of the reference engine's
``Backend`` / ``ModelForward`` surface over that ABI, used by the tests and the benchmark.
There is no CPU fallback: every operator raises if the library or an sm_100 device is missing.
"""
from .capi import OranguError, lib_path, load  # noqa: F401
from .backend import CudaBackend, QuantMatrix, MatmulOp  # noqa: F401
from .model import LlamaModel, KvCache  # noqa: F401
from .scheduler import SlotPool, SlotGuard  # noqa: F401

GGML_TYPE_F32, GGML_TYPE_Q8_0, GGML_TYPE_Q4_K, GGML_TYPE_Q6_K = 0, 8, 12, 14

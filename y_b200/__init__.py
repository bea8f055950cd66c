"""y_b200: B200 (sm_100a) kernels for the quantised-inference GEMM path.

`y_b200._lib` binds the C ABI (include/y_b200.h) of liby_b200.so; `y_b200.quant`
is the operator layer on torch CUDA tensors; `y_b200.runtime` mirrors the
reference's host launch API. There is no CPU or PyTorch fallback anywhere.
"""
from . import _lib  # noqa: F401  (fails loudly when the shared library is missing)

__all__ = ["_lib", "quant"]

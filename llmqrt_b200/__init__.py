"""llmqrt_b200: sm_100a kernels for quantized linear layers and KV-cache attention.

Importing the package loads (building it first if necessary) the CUDA library; there is no
CPU or eager fallback.
"""
from . import _lib  # noqa: F401  (fails loudly when the CUDA library is missing)

__all__ = ["_lib"]

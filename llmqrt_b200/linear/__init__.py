"""Quantized linear layers and the method registry (ref: runtime/nn_models/modules/linear/__init__.py:5-13)."""
from .linear_awq import WQLinear_GEMM
from .linear_base import LinearBase
from .linear_fp8 import FP8DynamicLinear, FP8StaticLinear
from .linear_sq import SqW8A8BBF16OBF16PerChannel, SqW8A8BBF16OBF16PerTensor

method_to_linear: dict[str, type[LinearBase]] = {
    "awq": WQLinear_GEMM,
    "sq": SqW8A8BBF16OBF16PerTensor,
    "fp8_static_quant": FP8StaticLinear,
    "fp8_dynamic_quant": FP8DynamicLinear,
}


def get_concrete_linear_module(quant_method):
    return method_to_linear[quant_method]


__all__ = ["LinearBase", "WQLinear_GEMM", "FP8DynamicLinear", "FP8StaticLinear", "SqW8A8BBF16OBF16PerTensor",
           "SqW8A8BBF16OBF16PerChannel", "method_to_linear", "get_concrete_linear_module"]

"""llmqrt_b200: sm_100a kernels for quantized linear layers and KV-cache attention.

Importing the package loads (building it first if necessary) the CUDA library; there is no
CPU or eager fallback.
"""
from __future__ import annotations

import importlib
import importlib.util
import sys
import types

from . import _lib  # noqa: F401  (fails loudly when the CUDA library is missing)

__all__ = ["_lib", "install_reference_aliases"]

# reference module name -> module of this package that stands in for it
_ALIASES = {
    "sq_fp8_kernels": "llmqrt_b200.sq_fp8_kernels",                    # runtime/csrc/bindings.cpp:7-14
    "triton_kernels.awq_kernels": "llmqrt_b200.triton_kernels.awq_kernels",   # runtime/triton_kernels/awq_kernels.py
}


def install_reference_aliases(package: str = "runtime", flash_attn: bool = False) -> list[str]:
    """Presents this package's kernels under the module names the reference's callers import.

    After the call
        from runtime.sq_fp8_kernels import w8a8_int8_linear_bbf16_obf16_per_tensor,
            cutlass_f8f8bf16_tensorwise_sm89, cutlass_f8f8bf16_rowwise_sm89
        from runtime.triton_kernels.awq_kernels import awq_gemm_triton, awq_dequantize_triton
    (the imports of runtime/nn_models/modules/linear/linear_sq.py:14, linear_fp8.py:7-8,
    linear_awq.py:14 and of the three files under runtime/unittest) resolve to the sm_100a kernels.
    If a package called `package` is importable (the reference checked out on sys.path) the aliases
    are attached to it and its own pure-Python modules stay reachable; otherwise an empty stand-in
    package is registered.  flash_attn=True also registers this package's attention module as
    `flash_attn` (the import at runtime/nn_models/modules/nonlinear/attn.py:11) -- only when no real
    flash_attn has been imported yet.  Returns the module names that were registered.
    """
    done = []
    root = sys.modules.get(package)
    if root is None:
        try:
            found = importlib.util.find_spec(package) is not None
        except (ImportError, ValueError):
            found = False
        if found:
            root = importlib.import_module(package)
        else:
            root = types.ModuleType(package)
            root.__path__ = []                                   # marks it as a package
            sys.modules[package] = root
            done.append(package)
    for ref_name, ours in _ALIASES.items():
        mod = importlib.import_module(ours)
        parent = root
        parts = ref_name.split(".")
        for i, part in enumerate(parts[:-1]):                    # intermediate packages
            full = ".".join([package] + parts[:i + 1])
            sub = sys.modules.get(full)
            if sub is None:
                try:
                    sub = importlib.import_module(full)
                except Exception:
                    sub = types.ModuleType(full)
                    sub.__path__ = []
                    sys.modules[full] = sub
                    done.append(full)
            setattr(parent, part, sub)
            parent = sub
        full = package + "." + ref_name
        sys.modules[full] = mod
        setattr(parent, parts[-1], mod)
        done.append(full)
    if flash_attn and "flash_attn" not in sys.modules:
        from . import attention
        sys.modules["flash_attn"] = attention
        done.append("flash_attn")
    return done

"""Drop-in for the reference's compiled extension module `runtime.sq_fp8_kernels`.

Same three functions, same positional arguments and results as the pybind module built from
runtime/csrc/bindings.cpp:7-14, plus the per-channel int8 entry point that the reference declares in
runtime/csrc/smoothquant/sq_gemm.h:19-24 but never compiled.  Differences that a caller can observe:
launches go to torch's current stream (the reference uses the legacy default stream for two of the
three), `alpha` may stay a CUDA tensor (it is read on the device instead of being synchronised to a
Python float), and any compute capability check is gone -- the kernels exist for sm_100a only.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops

_F8 = (torch.float8_e4m3fn, torch.float8_e5m2)


def _weight_nk(weight: torch.Tensor, what: str) -> torch.Tensor:
    """The callers pass W as a [K, N] view with stride [1, K] (`.t()` of the stored [N, K] weight,
    runtime/nn_models/modules/linear/linear_sq.py:128); recover the [N, K] row-major tensor."""
    if weight.dim() != 2:
        raise RuntimeError(f"{what}: weight must be 2-D")
    if weight.stride(0) != 1:
        raise RuntimeError(f"{what}: weight must be column-major [K, N] (stride(0) == 1)")
    return weight.t()


def _check_act(a: torch.Tensor, w_kn: torch.Tensor, what: str) -> None:
    if not a.is_cuda or a.device != w_kn.device:
        raise RuntimeError(f"{what}: input and weight must be CUDA tensors on the same device")
    if a.dim() != 2 or a.shape[1] != w_kn.shape[0]:
        raise RuntimeError(f"{what}: input [M, K] and weight [K, N] do not match")
    if a.stride(1) != 1 or a.stride(0) < a.shape[1]:
        raise RuntimeError(f"{what}: input must be row-major")


def w8a8_int8_linear_bbf16_obf16_per_tensor(input: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor,
                                           alpha, beta) -> torch.Tensor:
    """fp16 [M, N] = alpha * (int8 input [M, K] @ int8 weight [K, N]) + beta * bias[N].
    ref: runtime/csrc/smoothquant/sq_gemm.cu:36-160."""
    what = "w8a8_int8_linear_bbf16_obf16_per_tensor"
    _check_act(input, weight, what)
    if input.dtype != torch.int8 or weight.dtype != torch.int8:
        raise RuntimeError(f"{what}: input and weight must be int8")
    if bias is None:
        raise RuntimeError(f"{what}: bias is required")
    if input.shape[0] == 0:
        return torch.empty((0, weight.shape[1]), dtype=torch.float16, device=input.device)
    return ops.int8_linear_per_tensor(input, _weight_nk(weight, what), bias.to(input.device, torch.float16), alpha,
                                      float(beta))


def w8a8_int8_linear_bbf16_obf16_per_channel(input: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                                            alpha: torch.Tensor, beta: torch.Tensor,
                                            out_dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """[M, N] = (acc * beta[n]) * alpha[m] + bias[n]: alpha is the per-token activation scale [M] or [M, 1],
    beta the per-output-channel weight scale [N].  ref: declaration runtime/csrc/smoothquant/sq_gemm.h:19-24."""
    what = "w8a8_int8_linear_bbf16_obf16_per_channel"
    _check_act(input, weight, what)
    if input.dtype != torch.int8 or weight.dtype != torch.int8:
        raise RuntimeError(f"{what}: input and weight must be int8")
    if input.shape[0] == 0:
        return torch.empty((0, weight.shape[1]), dtype=out_dtype, device=input.device)
    return ops.int8_linear_per_channel(input, _weight_nk(weight, what), bias, alpha, beta, out_dtype)


def cutlass_f8f8bf16_tensorwise_sm89(XQ: torch.Tensor, WQ: torch.Tensor, bias: Optional[torch.Tensor], alpha, beta,
                                     dtype_str: str) -> torch.Tensor:
    """T [M, N] = alpha * (fp8 XQ [M, K] @ e4m3 WQ [K, N]) + beta * bias, T from dtype_str.
    ref: runtime/csrc/fp8/sm89_fp8_tensorwise_cutlassgemm.cu:316-334 (checks :264-303, dtype :236-261)."""
    what = "cutlass_f8f8bf16_tensorwise_sm89"
    _check_act(XQ, WQ, what)
    if XQ.dtype not in _F8 or WQ.dtype != torch.float8_e4m3fn:
        raise RuntimeError(f"{what}: XQ must be e4m3/e5m2 and WQ e4m3")
    try:
        out_dtype = {"bfloat16": torch.bfloat16, "float16": torch.float16}[dtype_str]
    except KeyError:
        raise RuntimeError(f"{what}: dtype_str must be 'bfloat16' or 'float16'") from None
    if bias is not None:
        if bias.dim() != 1 or bias.shape[0] != WQ.shape[1] or bias.dtype not in (torch.float16, torch.bfloat16):
            raise RuntimeError(f"{what}: bias must be a 16-bit [N] vector")
        bias = bias.to(out_dtype)
    if XQ.shape[0] == 0:
        return torch.empty((0, WQ.shape[1]), dtype=out_dtype, device=XQ.device)
    return ops.fp8_linear_tensorwise(XQ, _weight_nk(WQ, what), bias, alpha, float(beta), out_dtype)


def cutlass_f8f8bf16_rowwise_sm89(XQ: torch.Tensor, WQ: torch.Tensor, bias: Optional[torch.Tensor],
                                  x_scale: torch.Tensor, w_scale: torch.Tensor, use_fast_accum: bool) -> torch.Tensor:
    """bf16 [M, N] = ((XQ @ WQ) * x_scale[M,1]) * w_scale[1,N] + bias.  `use_fast_accum` is accepted and
    ignored: both settings select the same fp32-accumulating instruction in the reference.
    ref: runtime/csrc/fp8/sm89_fp8_rowwise_fbgemm.cu:582-606 (checks :526-566)."""
    what = "cutlass_f8f8bf16_rowwise_sm89"
    _check_act(XQ, WQ, what)
    if XQ.dtype not in _F8 or WQ.dtype != torch.float8_e4m3fn:
        raise RuntimeError(f"{what}: XQ must be e4m3/e5m2 and WQ e4m3")
    M, N = XQ.shape[0], WQ.shape[1]
    if x_scale.dtype != torch.float32 or w_scale.dtype != torch.float32:
        raise RuntimeError(f"{what}: scales must be fp32")
    if tuple(x_scale.shape) != (M, 1) or tuple(w_scale.shape) != (1, N):
        raise RuntimeError(f"{what}: Expected x_scale [M, 1] and w_scale [1, N], got {tuple(x_scale.shape)} "
                           f"and {tuple(w_scale.shape)}")
    if bias is not None and (bias.dim() != 1 or bias.shape[0] != N or bias.dtype not in (torch.bfloat16, torch.float32)):
        raise RuntimeError(f"{what}: bias must be a bf16 or fp32 [N] vector")
    if M == 0:
        return torch.empty((0, N), dtype=torch.bfloat16, device=XQ.device)
    return ops.fp8_linear_rowwise(XQ, _weight_nk(WQ, what), bias, x_scale.contiguous(), w_scale.contiguous())

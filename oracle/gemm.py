"""W8A8 GEMMs and their epilogues (test oracle; see oracle/__init__.py)."""
from __future__ import annotations

import numpy as np
import torch


def _fma32(a: np.ndarray, b: np.ndarray, c: np.ndarray) -> np.ndarray:
    """fp32 fused multiply-add emulated through fp64.

    The product of two fp32 numbers is exact in fp64; the sum is rounded once
    to 53 bits and once more to 24 bits, which differs from a true fma only on
    exact double-rounding ties.
    """
    return (a.astype(np.float64) * b.astype(np.float64) + c.astype(np.float64)).astype(np.float32)


def int8_accumulate(a_q: torch.Tensor, w_q: torch.Tensor) -> torch.Tensor:
    """Exact int32 accumulators  acc[m, n] = sum_k a_q[m, k] * w_q[n, k].

    a_q int8 [M, K], w_q int8 [N, K] (the reference passes the same memory as
    a [K, N] view with stride [1, K], runtime/nn_models/modules/linear/linear_sq.py:128).
    Computed in fp64 BLAS: |sum| <= 128*128*K < 2**53, so every partial sum is
    exact.  Follows the s8 x s8 -> s32 tensor-op GEMM of
    runtime/csrc/smoothquant/sq_gemm.cu:36-76.
    """
    acc = a_q.to(torch.float64) @ w_q.to(torch.float64).t()
    return acc.to(torch.int32)


def int8_linear_per_tensor(a_q, w_q, bias, alpha: float, beta: float) -> torch.Tensor:
    """out = fp16( alpha * float(acc) + beta * float(bias) ).

    Follows runtime/csrc/smoothquant/sq_gemm.cu:36-160: the broadcast bias is
    both source C and destination D (:112, :125-131) and the epilogue is
    LinearCombination<half, 8, int32, float> (:73-75), whose arithmetic is
    t = beta * C; D = fma(alpha, acc, t) in fp32, rounded to nearest fp16
    (3rdparty/cutlass/include/cutlass/epilogue/thread/linear_combination.h:219-251).
    """
    acc = int8_accumulate(a_q, w_q).numpy().astype(np.float32)
    c = bias.to(torch.float32).numpy().reshape(1, -1)
    t = (np.float32(beta) * c).astype(np.float32)
    d = _fma32(np.broadcast_to(np.float32(alpha), acc.shape), acc, np.broadcast_to(t, acc.shape))
    return torch.from_numpy(d).to(torch.float16)


def dequant_per_token_per_channel(acc, w_scale, a_scale, bias, out_dtype) -> torch.Tensor:
    """out = T( (float(acc) * w_scale[n]) * a_scale[m]  [+ float(bias[n])] ).

    Follows dequantize_activation_w_per_channel_a_per_token,
    runtime/utils/quantization_utils.py:90-97 (fp32, weight scale first, then
    the token scale, one rounding to the 16-bit type).  The reference function
    has no bias; the optional bias add is the fp32 add of the row-wise fp8
    epilogue (runtime/csrc/fp8/sm89_fp8_rowwise_fbgemm.cu:224-232).
    """
    f = acc.to(torch.float32)
    f = f * w_scale.to(torch.float32).reshape(1, -1)
    f = f * a_scale.to(torch.float32).reshape(-1, 1)
    if bias is not None:
        f = f + bias.to(torch.float32).reshape(1, -1)
    return f.to(out_dtype)


def int8_linear_per_channel(a_q, w_q, bias, a_scale, w_scale, out_dtype=torch.float16):
    """Per-token x per-channel W8A8 linear: exact int32 GEMM + fused dequant.

    This is the entry point declared (but never implemented) in
    runtime/csrc/smoothquant/sq_gemm.h:19-24.
    """
    return dequant_per_token_per_channel(int8_accumulate(a_q, w_q), w_scale, a_scale, bias, out_dtype)


def fp8_accumulate(a_q: torch.Tensor, w_q: torch.Tensor) -> torch.Tensor:
    """fp32 view of the fp8 GEMM accumulators, computed in fp64.

    a_q: e4m3 or e5m2 [M, K]; w_q: e4m3 [N, K].  Products of two fp8 numbers
    are exact in fp32; the reference accumulates them in fp32 inside the tensor
    core (runtime/csrc/fp8/sm89_fp8_rowwise_fbgemm.cu:147-150) in a
    hardware-defined order, so the oracle gives the infinitely precise sum
    rounded once and comparisons are tolerance-based.
    """
    acc = a_q.to(torch.float64) @ w_q.to(torch.float64).t()
    return acc.to(torch.float32)


def fp8_linear_rowwise(a_q, w_q, bias, x_scale, w_scale) -> torch.Tensor:
    """out = bf16( ((acc * x_scale[m]) * w_scale[n]) + float(bias[n] or 0) ).

    Follows the epilogue visitor tree of
    runtime/csrc/fp8/sm89_fp8_rowwise_fbgemm.cu:193-245 (Accum -> *XScale ->
    *WScale -> +Bias -> store), every node rounding to nearest in fp32; output
    is always bf16 (:75).  x_scale fp32 [M,1], w_scale fp32 [1,N].
    """
    f = fp8_accumulate(a_q, w_q)
    f = f * x_scale.to(torch.float32).reshape(-1, 1)
    f = f * w_scale.to(torch.float32).reshape(1, -1)
    if bias is not None:
        f = f + bias.to(torch.float32).reshape(1, -1)
    return f.to(torch.bfloat16)


def fp8_linear_tensorwise(a_q, w_q, bias, alpha: float, beta: float, out_dtype) -> torch.Tensor:
    """out = T( alpha * acc + beta * float(bias or 0) ), T in {bf16, fp16}.

    Follows runtime/csrc/fp8/sm89_fp8_tensorwise_cutlassgemm.cu:23-163: same
    LinearCombination epilogue as the int8 kernel (:61-63), a missing bias is
    replaced by zeros (:101-107).
    """
    acc = fp8_accumulate(a_q, w_q).numpy()
    n = acc.shape[1]
    c = (bias.to(torch.float32).numpy() if bias is not None else np.zeros(n, np.float32)).reshape(1, -1)
    t = (np.float32(beta) * c).astype(np.float32)
    d = _fma32(np.broadcast_to(np.float32(alpha), acc.shape), acc, np.broadcast_to(t, acc.shape))
    return torch.from_numpy(d).to(out_dtype)

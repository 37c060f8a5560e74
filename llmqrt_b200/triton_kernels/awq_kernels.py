"""Drop-in for the reference module `runtime.triton_kernels.awq_kernels` -- CUDA behind, no Triton.

`awq_gemm_triton` and `awq_dequantize_triton` keep the reference's names, argument order and tensor
layouts (runtime/triton_kernels/awq_kernels.py:273-279 and :328-337).  The tuning arguments
(split_k_iters, block sizes) are accepted and validated like the reference's but do not steer the CUDA
kernels, which pick their own decomposition.
"""
from __future__ import annotations

import torch

from .. import ops

AWQ_TRITON_SUPPORTED_GROUP_SIZES = [-1, 32, 64, 128]


def _check_layer(qweight, scales, zeros):
    K = qweight.shape[0]
    N = scales.shape[1]
    group_size = K // scales.shape[0]
    assert K > 0 and N > 0
    assert qweight.shape[1] == N // 8
    assert scales.shape[0] == K // group_size and zeros.shape[0] == K // group_size and zeros.shape[1] == N // 8
    assert group_size <= K
    assert group_size in AWQ_TRITON_SUPPORTED_GROUP_SIZES or group_size == K
    return K, N, group_size


def awq_dequantize_triton(qweight: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, block_size_x: int = 32,
                          block_size_y: int = 32) -> torch.Tensor:
    """W[K, N] = (nibble(qweight) - nibble(zeros)) * scales, in scales.dtype."""
    _check_layer(qweight, scales, zeros)
    return ops.awq_dequantize(qweight, scales, zeros)


def awq_gemm_triton(input: torch.Tensor, qweight: torch.Tensor, scales: torch.Tensor, qzeros: torch.Tensor,
                    split_k_iters: int, block_size_m: int = 32, block_size_n: int = 32,
                    block_size_k: int = 32) -> torch.Tensor:
    """C[M, N] = input[M, K] @ dequant(qweight), in scales.dtype.

    The layer is repacked into the streaming layout on every call, which costs one extra pass over the
    4-bit weights; callers that own the layer (the WQLinear_GEMM module) repack once and keep it.
    """
    M, K = input.shape
    K2, N, _ = _check_layer(qweight, scales, qzeros)
    assert M > 0 and K2 == K
    assert split_k_iters & (split_k_iters - 1) == 0 and split_k_iters != 0
    assert split_k_iters <= 32
    packed = ops.AwqPacked(qweight, scales, qzeros)
    out = ops.awq_gemm(input.to(torch.float16), packed)
    return out if scales.dtype == torch.float16 else out.to(scales.dtype)

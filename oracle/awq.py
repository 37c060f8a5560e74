"""AWQ W4A16 packing, dequantization and GEMM (test oracle; see oracle/__init__.py)."""
from __future__ import annotations

import numpy as np
import torch

# Nibble i of a packed int32 holds logical column 8*j + PACK_ORDER[i]
# (runtime/nn_models/modules/linear/linear_awq.py:192-201).
PACK_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)


def pack_cols(vals: torch.Tensor) -> torch.Tensor:
    """Pack uint4 values [R, N] into int32 [R, N/8] in the AWQ nibble order.

    Follows the packing loop of linear_awq.py:186-201 (weights) and :205-218
    (zero points).
    """
    v = vals.to(torch.int64).reshape(vals.shape[0], -1, 8)
    out = torch.zeros(v.shape[:2], dtype=torch.int64)
    for i, src in enumerate(PACK_ORDER):
        out |= (v[:, :, src] & 0xF) << (4 * i)
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out)
    return out.to(torch.int32)


def unpack_cols(packed: torch.Tensor) -> torch.Tensor:
    """Inverse of pack_cols: int32 [R, N/8] -> uint4 values [R, N] (int32).

    Follows unpack_awq + reverse_awq_order + the 0xF mask,
    runtime/utils/packing_utils.py:8-45, 72-73.
    """
    p = packed.to(torch.int64) & 0xFFFFFFFF
    out = torch.empty(packed.shape[0], packed.shape[1], 8, dtype=torch.int32)
    for i, dst in enumerate(PACK_ORDER):
        out[:, :, dst] = ((p >> (4 * i)) & 0xF).to(torch.int32)
    return out.reshape(packed.shape[0], -1)


def dequantize(qweight, qzeros, scales, group_size: int) -> torch.Tensor:
    """W[K, N] = (nibble(qweight) - nibble(qzeros[k // G])) * scales[k // G].

    Follows dequantize_gemm, runtime/utils/packing_utils.py:65-80, and the
    Triton kernel runtime/triton_kernels/awq_kernels.py:33-127: the integer
    difference is converted to the scale dtype and multiplied there, i.e. one
    rounding to fp16.
    """
    w = unpack_cols(qweight)
    z = unpack_cols(qzeros).repeat_interleave(group_size, dim=0)
    s = scales.repeat_interleave(group_size, dim=0)
    return ((w - z).to(torch.float32) * s.to(torch.float32)).to(scales.dtype)


def gemm(x, qweight, qzeros, scales, group_size: int) -> torch.Tensor:
    """C[M, N] = x[M, K] @ dequantize(...), result in the scale dtype.

    Follows runtime/triton_kernels/awq_kernels.py:134-267.  The reference
    accumulates in fp16 with a split-K atomic add (:160-168, :264-267), which
    is order dependent; the oracle accumulates exactly (fp64) and rounds once,
    so comparisons with it are tolerance-based.
    """
    w = dequantize(qweight, qzeros, scales, group_size).to(torch.float64)
    return (x.to(torch.float64) @ w).to(scales.dtype)


def random_layer(K: int, N: int, group_size: int, seed: int):
    """Seeded synthetic AWQ layer: uint4 weights and zero points ~U{0..15},
    fp16 scales ~U(0.001, 0.02), packed as the reference stores them
    (buffer shapes of linear_awq.py:97-131)."""
    g = torch.Generator().manual_seed(seed)
    w = torch.randint(0, 16, (K, N), generator=g, dtype=torch.int32)
    z = torch.randint(0, 16, (K // group_size, N), generator=g, dtype=torch.int32)
    s = (torch.rand(K // group_size, N, generator=g) * 0.019 + 0.001).to(torch.float16)
    return pack_cols(w), pack_cols(z), s


def repack_k_major(qweight: torch.Tensor) -> np.ndarray:
    """Expected output of the load-time repack into the streaming layout.

    Result uint32 [N, K/8]: word (n, j) holds the eight K-consecutive values
    w[8j .. 8j+7, n] with value 2p in nibble p and value 2p+1 in nibble p+4,
    so that `(word >> 4p) & 0x000F000F` yields the pair (2p, 2p+1) in the two
    halves of a half2.
    """
    w = unpack_cols(qweight).numpy().astype(np.uint32)          # [K, N]
    K, N = w.shape
    wt = w.T.reshape(N, K // 8, 8)
    out = np.zeros((N, K // 8), dtype=np.uint32)
    for p in range(4):
        out |= wt[:, :, 2 * p] << np.uint32(4 * p)
        out |= wt[:, :, 2 * p + 1] << np.uint32(4 * p + 16)
    return out

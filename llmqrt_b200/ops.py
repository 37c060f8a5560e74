"""Tensor-level wrappers over the C ABI: allocate outputs with torch, pass raw pointers down.

Every function launches on torch's current stream of the tensors' device and never synchronises.
"""
from __future__ import annotations

import torch

from . import _lib as L

F8 = torch.float8_e4m3fn


def _rows(x: torch.Tensor) -> torch.Tensor:
    """View [..., K] as a 2-D [M, K] tensor with unit inner stride (copying only if it must)."""
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    return x2


# ---------------------------------------------------------------------------------------------
# activation quantizers
# ---------------------------------------------------------------------------------------------
def quantize_int8(x: torch.Tensor, per_token: bool, scale_mul: float = 1.0):
    """Returns (q int8 [M,K], scale in x.dtype ([M,1] or 0-d), scale_f32 ([M] or [1]) = T(scale*scale_mul))."""
    dev = L.require_cuda(x)
    x2 = _rows(x)
    M, K = x2.shape
    q = torch.empty((M, K), dtype=torch.int8, device=dev)
    n = M if per_token else 1
    scale = torch.empty(n, dtype=x.dtype, device=dev)
    scale_f32 = torch.empty(n, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        L.call("llmqrt_quantize_int8", L.ptr(x2), L.dtype_code(x.dtype), M, K, x2.stride(0), int(per_token),
               L.ptr(q), L.ptr(scale), L.ptr(scale_f32), float(scale_mul), L.ptr(L.workspace(dev)), L.stream(dev))
    return q, (scale.reshape(M, 1) if per_token else scale.reshape(())), scale_f32


def quantize_fp8(x: torch.Tensor, per_token: bool, scale_mul: float = 1.0):
    """Returns (q e4m3 [M,K], scale_f32 ([M,1] or [1]) = float(scale) * scale_mul)."""
    dev = L.require_cuda(x)
    x2 = _rows(x)
    M, K = x2.shape
    q = torch.empty((M, K), dtype=F8, device=dev)
    n = M if per_token else 1
    scale_f32 = torch.empty(n, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        L.call("llmqrt_quantize_fp8", L.ptr(x2), L.dtype_code(x.dtype), M, K, x2.stride(0), int(per_token),
               L.ptr(q), L.ptr(scale_f32), float(scale_mul), L.ptr(L.workspace(dev)), L.stream(dev))
    return q, (scale_f32.reshape(M, 1) if per_token else scale_f32)


def quantize_fp8_static(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    dev = L.require_cuda(x, scale)
    x2 = _rows(x)
    M, K = x2.shape
    q = torch.empty((M, K), dtype=F8, device=dev)
    s = scale.to(torch.float32).reshape(-1)
    with torch.cuda.device(dev):
        L.call("llmqrt_quantize_fp8_static", L.ptr(x2), L.dtype_code(x.dtype), M, K, x2.stride(0), L.ptr(s),
               L.ptr(q), L.stream(dev))
    return q


# ---------------------------------------------------------------------------------------------
# W8A8 GEMMs.  `w` is always the [N, K] row-major weight.
#
# static_weight=True tells the kernel that `w` is a stored weight that nothing queued on the stream
# writes; it may then fetch the first weight tiles while the preceding kernel is still running.  The
# default waits for the preceding kernel before reading anything, so quantizing `w` on the same
# stream right before the call is safe.  The Linear modules and the decoder, whose weights are
# buffers prepared long before, pass True.
# ---------------------------------------------------------------------------------------------
def _flags(static_weight: bool) -> int:
    return L.GEMM_STATIC_WEIGHT if static_weight else 0


def _alpha_args(alpha, dev):
    """A Python number travels by value; a tensor is read on the device (no host sync)."""
    if isinstance(alpha, torch.Tensor):
        a = alpha.to(device=dev, dtype=torch.float32).reshape(-1)
        if a.numel() != 1:
            raise RuntimeError("alpha must be a scalar")
        return 0.0, a
    return float(alpha), None


def int8_linear_per_tensor(a, w, bias, alpha, beta: float, static_weight: bool = False) -> torch.Tensor:
    dev = L.require_cuda(a, w, bias)
    M, K = a.shape
    N = w.shape[0]
    out = torch.empty((M, N), dtype=torch.float16, device=dev)
    av, ad = _alpha_args(alpha, dev)
    with torch.cuda.device(dev):
        L.call("llmqrt_w8a8_int8_linear_per_tensor", L.ptr(a), a.stride(0), L.ptr(w), w.stride(0), L.ptr(bias), av,
               L.ptr(ad), float(beta), L.ptr(out), N, M, N, K, L.ptr(L.workspace(dev)), L.stream(dev),
               _flags(static_weight))
    return out


def int8_linear_per_channel(a, w, bias, a_scale, w_scale, out_dtype, static_weight: bool = False) -> torch.Tensor:
    dev = L.require_cuda(a, w, bias, a_scale, w_scale)
    M, K = a.shape
    N = w.shape[0]
    out = torch.empty((M, N), dtype=out_dtype, device=dev)
    a_s = a_scale.to(torch.float32).reshape(-1).contiguous()
    w_s = w_scale.to(torch.float32).reshape(-1).contiguous()
    if a_s.numel() != M or w_s.numel() != N:
        raise RuntimeError("per-channel int8 linear: a_scale must have M elements and w_scale N elements")
    with torch.cuda.device(dev):
        L.call("llmqrt_w8a8_int8_linear_per_channel", L.ptr(a), a.stride(0), L.ptr(w), w.stride(0), L.ptr(bias),
               L.dtype_code(bias.dtype) if bias is not None else L.F16, L.ptr(a_s), L.ptr(w_s), L.ptr(out),
               L.dtype_code(out_dtype), N, M, N, K, L.ptr(L.workspace(dev)), L.stream(dev), _flags(static_weight))
    return out


def int8_gemm_s32(a, w, static_weight: bool = False) -> torch.Tensor:
    dev = L.require_cuda(a, w)
    M, K = a.shape
    N = w.shape[0]
    out = torch.empty((M, N), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        L.call("llmqrt_w8a8_int8_gemm_s32", L.ptr(a), a.stride(0), L.ptr(w), w.stride(0), L.ptr(out), N, M, N, K,
               L.ptr(L.workspace(dev)), L.stream(dev), _flags(static_weight))
    return out


def fp8_linear_tensorwise(a, w, bias, alpha, beta: float, out_dtype, static_weight: bool = False) -> torch.Tensor:
    dev = L.require_cuda(a, w, bias)
    M, K = a.shape
    N = w.shape[0]
    out = torch.empty((M, N), dtype=out_dtype, device=dev)
    av, ad = _alpha_args(alpha, dev)
    with torch.cuda.device(dev):
        L.call("llmqrt_f8f8_tensorwise", L.ptr(a), L.dtype_code(a.dtype), a.stride(0), L.ptr(w), w.stride(0),
               L.ptr(bias), av, L.ptr(ad), float(beta), L.ptr(out), L.dtype_code(out_dtype), N, M, N, K,
               L.ptr(L.workspace(dev)), L.stream(dev), _flags(static_weight))
    return out


def fp8_linear_rowwise(a, w, bias, x_scale, w_scale, static_weight: bool = False) -> torch.Tensor:
    dev = L.require_cuda(a, w, bias, x_scale, w_scale)
    M, K = a.shape
    N = w.shape[0]
    out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    xs = x_scale.reshape(-1)
    ws = w_scale.reshape(-1)
    with torch.cuda.device(dev):
        L.call("llmqrt_f8f8bf16_rowwise", L.ptr(a), L.dtype_code(a.dtype), a.stride(0), L.ptr(w), w.stride(0),
               L.ptr(bias), L.dtype_code(bias.dtype) if bias is not None else L.BF16, L.ptr(xs), L.ptr(ws),
               L.ptr(out), N, M, N, K, L.ptr(L.workspace(dev)), L.stream(dev), _flags(static_weight))
    return out


def gemm_16bit(a, w, bias=None) -> torch.Tensor:
    """out[M,N] = a[M,K] @ w[N,K]^T (+ bias) on tcgen05, fp32 accumulate; a, w, bias share one 16-bit dtype."""
    dev = L.require_cuda(a, w, bias)
    M, K = a.shape
    N = w.shape[0]
    out = torch.empty((M, N), dtype=a.dtype, device=dev)
    with torch.cuda.device(dev):
        L.call("llmqrt_gemm_16bit", L.ptr(a), a.stride(0), L.ptr(w), w.stride(0), L.ptr(bias), L.ptr(out), N,
               L.dtype_code(a.dtype), M, N, K, L.ptr(L.workspace(dev)), L.stream(dev))
    return out


# ---------------------------------------------------------------------------------------------
# AWQ W4A16
# ---------------------------------------------------------------------------------------------
def awq_dequantize(qweight, scales, qzeros) -> torch.Tensor:
    """W[K, N] in scales.dtype from the reference storage layout."""
    dev = L.require_cuda(qweight, scales, qzeros)
    K, N = qweight.shape[0], scales.shape[1]
    G = K // scales.shape[0]
    out = torch.empty((K, N), dtype=torch.float16, device=dev)
    sc = scales if scales.dtype == torch.float16 else scales.to(torch.float16)
    with torch.cuda.device(dev):
        L.call("llmqrt_awq_dequantize", L.ptr(qweight.contiguous()), L.ptr(sc.contiguous()),
               L.ptr(qzeros.contiguous()), K, N, G, L.ptr(out), L.stream(dev))
    return out if scales.dtype == torch.float16 else out.to(scales.dtype)


class AwqPacked:
    """A layer repacked once into the K-major streaming layout (see llmqrt_awq_repack)."""

    __slots__ = ("wq_t", "sz_t", "K", "N", "G")

    def __init__(self, qweight, scales, qzeros):
        dev = L.require_cuda(qweight, scales, qzeros)
        self.K, self.N = int(qweight.shape[0]), int(scales.shape[1])
        self.G = self.K // int(scales.shape[0])
        self.wq_t = torch.empty((self.N, self.K // 8), dtype=torch.int32, device=dev)
        self.sz_t = torch.empty((self.N, self.K // self.G), dtype=torch.int32, device=dev)
        with torch.cuda.device(dev):
            L.call("llmqrt_awq_repack", L.ptr(qweight.contiguous()), L.ptr(scales.to(torch.float16).contiguous()),
                   L.ptr(qzeros.contiguous()), self.K, self.N, self.G, L.ptr(self.wq_t), L.ptr(self.sz_t),
                   L.stream(dev))


def awq_dequantize_t(packed: AwqPacked) -> torch.Tensor:
    """W^T[N, K] fp16 (K contiguous) from a repacked layer."""
    dev = packed.wq_t.device
    out = torch.empty((packed.N, packed.K), dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        L.call("llmqrt_awq_dequantize_t", L.ptr(packed.wq_t), L.ptr(packed.sz_t), packed.K, packed.N, packed.G,
               L.ptr(out), L.stream(dev))
    return out


def awq_gemm(x: torch.Tensor, packed: AwqPacked, bias=None) -> torch.Tensor:
    """C[M, N] fp16 = x[M, K] fp16 @ dequant(W) (+ bias): one fused kernel below 1024 tokens (a weight-streaming
    mma.sync kernel up to 64, the tcgen05 GEMM with in-kernel dequantization above); from 1024 tokens on the
    weights are expanded panel-wise into the workspace and multiplied by the two-CTA fp16 kernel."""
    dev = L.require_cuda(x, packed.wq_t, bias)
    x2 = _rows(x)
    M, K = x2.shape
    if K != packed.K:
        raise RuntimeError(f"awq_gemm: x has K={K}, layer has K={packed.K}")
    out = torch.empty((M, packed.N), dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        L.call("llmqrt_awq_gemm", L.ptr(x2), x2.stride(0), L.ptr(packed.wq_t), L.ptr(packed.sz_t), L.ptr(bias),
               L.ptr(out), packed.N, M, packed.N, K, packed.G, L.ptr(L.workspace(dev)), L.stream(dev))
    return out

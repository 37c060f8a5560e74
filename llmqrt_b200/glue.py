"""Fused block-glue ops of the decode step: RMSNorm, rotary embedding + KV-cache write, SiLU*up."""
from __future__ import annotations

import torch

from . import _lib as L


def rmsnorm(x, weight, eps: float, residual=None, quantize: bool = False, want_y: bool = True, comm=None):
    """y = weight * T(x32 * rsqrt(mean(x32^2) + eps)) over the last dimension.

    residual: if given, h = x + residual (rounded to T) is normalised instead and also returned.
    quantize: also return the per-token int8 quantization (q, scale_f32[M]) of y.
    comm: a tp.PeerAllreduce; `residual` then holds this rank's tensor-parallel PARTIAL sums and is
          all-reduced over the group first -- inside the same kernel when it fits the communicator,
          else by NCCL (`residual` is then summed in place).  `residual` may also be the token returned
          by `comm.linear_push`: the GEMM has then sent the partial sums itself and this kernel only gathers.
    Returns (y or None, h or None, q or None, scale or None).
    """
    from .tp import PushedPartial
    pushed = isinstance(residual, PushedPartial)          # the partial sums are already on their way to the peers
    dev = L.require_cuda(x, weight, None if pushed else residual)
    H = x.shape[-1]
    x2 = x.reshape(-1, H).contiguous()
    M = x2.shape[0]
    if pushed:
        if comm is None or (residual.M, residual.H) != (M, H):
            raise RuntimeError("rmsnorm: pushed partial sums need their communicator and the same [M, H]")
        h = torch.empty_like(x2)
        y = torch.empty_like(x2) if want_y else None
        q = torch.empty((M, H), dtype=torch.int8, device=dev) if quantize else None
        s = torch.empty(M, dtype=torch.float32, device=dev) if quantize else None
        with torch.cuda.device(dev):
            L.call("llmqrt_comm_allreduce_rmsnorm", comm.handle, None, L.ptr(x2), L.ptr(h), L.ptr(weight),
                   float(eps), L.ptr(y), L.ptr(q), L.ptr(s), L.dtype_code(x.dtype), M, H, L.stream(dev))
        return (y.reshape(x.shape) if y is not None else None, h.reshape(x.shape), q, s)
    r2 = residual.reshape(-1, H).contiguous() if residual is not None else None
    if comm is not None and r2 is not None and r2.data_ptr() % 16:
        r2 = r2.clone()                                  # rank-local misalignment must not change the path
    h = torch.empty_like(x2) if residual is not None else None
    y = torch.empty_like(x2) if want_y else None
    q = torch.empty((M, H), dtype=torch.int8, device=dev) if quantize else None
    s = torch.empty(M, dtype=torch.float32, device=dev) if quantize else None
    fused = comm is not None and r2 is not None and comm.eligible(r2) and comm.fits_rows(M, H)
    if comm is not None and r2 is not None and not fused:
        torch.distributed.all_reduce(r2, group=comm.group)
    with torch.cuda.device(dev):
        if fused:
            L.call("llmqrt_comm_allreduce_rmsnorm", comm.handle, L.ptr(r2), L.ptr(x2), L.ptr(h), L.ptr(weight),
                   float(eps), L.ptr(y), L.ptr(q), L.ptr(s), L.dtype_code(x.dtype), M, H, L.stream(dev))
        else:
            L.call("llmqrt_rmsnorm", L.ptr(x2), L.ptr(r2), L.ptr(h), L.ptr(weight), float(eps), L.ptr(y), L.ptr(q),
                   L.ptr(s), L.dtype_code(x.dtype), M, H, L.stream(dev))
    shape = x.shape
    return (y.reshape(shape) if y is not None else None, h.reshape(shape) if h is not None else None, q, s)


def rope_tables(head_dim: int, max_seq_len: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    """cos / sin of pos * theta**(-2i/d), fp32 [max_seq_len, d/2], built on the CPU exactly like the
    reference's freqs_cis table (runtime/nn_models/modules/nonlinear/attn.py:37-43) and then moved."""
    freqs = 1.0 / (theta ** (torch.arange(0, head_dim, 2)[: head_dim // 2].float() / head_dim))
    ang = torch.outer(torch.arange(max_seq_len), freqs).float()
    return torch.cos(ang).to(device).contiguous(), torch.sin(ang).to(device).contiguous()


def rope_kv_write(q, k, v, cos, sin, pos0: int = 0, pos_dev=None, k_cache=None, v_cache=None):
    """Rotates q [B,S,Hq,d] and k [B,S,Hkv,d] IN PLACE at positions pos + s and, when caches are given,
    writes the rotated k and v into rows pos + s of the caches [Bc, Smax, Hkv, d]."""
    dev = L.require_cuda(q, k, v, cos, sin, pos_dev, k_cache, v_cache)
    B, S, Hq, d = q.shape
    Hkv = k.shape[2]
    for t in (q, k) + ((v,) if v is not None else ()):
        if t.stride(3) != 1 or t.stride(2) != d or t.stride(0) != S * t.stride(1):
            raise RuntimeError("rope_kv_write: tensors must be [B, S, H, d] with heads and d contiguous")
    if v is not None and v.stride(1) != k.stride(1):
        raise RuntimeError("rope_kv_write: k and v must share the token stride")
    with torch.cuda.device(dev):
        L.call("llmqrt_rope_kv_write", L.ptr(q), q.stride(1), L.ptr(k), L.ptr(v), k.stride(1), L.ptr(k_cache),
               L.ptr(v_cache), k_cache.stride(0) if k_cache is not None else 0,
               k_cache.stride(1) if k_cache is not None else 0, int(pos0), L.ptr(pos_dev), L.ptr(cos), L.ptr(sin),
               cos.shape[0], L.dtype_code(q.dtype), B, S, Hq, Hkv, d, L.stream(dev))


def silu_mul(gate_up, quantize: bool = False, want_y: bool = True):
    """h = silu(gate) * up for gate_up [..., 2I] (gate first).  Returns (h or None, q or None, scale or None)."""
    dev = L.require_cuda(gate_up)
    I = gate_up.shape[-1] // 2
    g2 = gate_up.reshape(-1, 2 * I)
    if g2.stride(1) != 1:
        g2 = g2.contiguous()
    M = g2.shape[0]
    y = torch.empty((M, I), dtype=gate_up.dtype, device=dev) if want_y else None
    q = torch.empty((M, I), dtype=torch.int8, device=dev) if quantize else None
    s = torch.empty(M, dtype=torch.float32, device=dev) if quantize else None
    with torch.cuda.device(dev):
        L.call("llmqrt_silu_mul", L.ptr(g2), g2.stride(0), L.ptr(y), L.ptr(q), L.ptr(s), L.dtype_code(gate_up.dtype),
               M, I, L.stream(dev))
    return (y.reshape(*gate_up.shape[:-1], I) if y is not None else None, q, s)

"""Attention entry points with the call signatures the reference uses from the flash-attn package.

`flash_attn_func` and `flash_attn_with_kvcache` accept the keyword subset of the reference's two
call sites (runtime/nn_models/modules/nonlinear/attn.py:290-298 and :305-315) and run this
package's own sm_100a kernels; arguments of the flash-attn API that the reference never sets are
accepted only at their neutral values.
"""
from __future__ import annotations

import math

import torch

from . import _lib as L


def _check_common(q, softmax_scale, dropout_p=0.0, window_size=(-1, -1), alibi_slopes=None):
    if dropout_p != 0.0:
        raise NotImplementedError("llmqrt_b200 attention: dropout is not supported (inference only)")
    if alibi_slopes is not None:
        raise NotImplementedError("llmqrt_b200 attention: ALiBi is not supported")
    if tuple(window_size) != (-1, -1):
        raise NotImplementedError("llmqrt_b200 attention: sliding windows are not supported")
    d = q.shape[-1]
    if softmax_scale is not None and not math.isclose(softmax_scale, d ** -0.5, rel_tol=1e-6):
        raise NotImplementedError("llmqrt_b200 attention: only the default softmax scale d**-0.5 is supported")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("llmqrt_b200 attention: q/k/v must be fp16 or bf16")


def _token_strided(x: torch.Tensor) -> torch.Tensor:
    """[B, S, H, d] with heads and d contiguous and batches back to back; copies only if it must."""
    B, S, H, d = x.shape
    if x.stride(3) == 1 and x.stride(2) == d and x.stride(0) == S * x.stride(1) and x.stride(1) % 8 == 0 \
            and x.data_ptr() % 16 == 0:
        return x
    return x.contiguous()


def flash_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1), softcap=0.0,
                    alibi_slopes=None, deterministic=False, return_attn_probs=False):
    """O = softmax(mask(Q K^T / sqrt(d))) V.  q [B,S,Hq,d]; k, v [B,S,Hkv,d]; returns [B,S,Hq,d]."""
    _check_common(q, softmax_scale, dropout_p, window_size, alibi_slopes)
    if return_attn_probs:
        raise NotImplementedError("llmqrt_b200 attention: attention probabilities are never materialised")
    dev = L.require_cuda(q, k, v)
    B, S, Hq, d = q.shape
    if k.shape[1] != S or v.shape != k.shape or k.shape[0] != B or k.shape[3] != d:
        raise RuntimeError("flash_attn_func: q, k, v must share batch, sequence length and head_dim")
    Hkv = k.shape[2]
    q, k, v = _token_strided(q), _token_strided(k), _token_strided(v)
    if k.stride(1) != v.stride(1):
        v = v.contiguous()
        k = k.contiguous()
    out = torch.empty((B, S, Hq, d), dtype=q.dtype, device=dev)
    with torch.cuda.device(dev):
        L.call("llmqrt_attn_prefill", L.ptr(q), q.stride(1), L.ptr(k), L.ptr(v), k.stride(1), L.ptr(out),
               out.stride(1), L.dtype_code(q.dtype), B, S, Hq, Hkv, d, int(bool(causal)), float(softcap),
               L.stream(dev))
    return out


def kv_append(k_cache, v_cache, k, v, cache_seqlens=None, start_pos: int = 0):
    """cache[b, pos_b + s] = k/v[b, s] with pos_b = cache_seqlens[b] (device int32) or `start_pos`."""
    dev = L.require_cuda(k_cache, v_cache, k, v, cache_seqlens)
    B, S_new, Hkv, d = k.shape
    if k_cache.stride(3) != 1 or k_cache.stride(2) != d or v_cache.stride() != k_cache.stride():
        raise RuntimeError("kv_append: caches must be [B, S, Hkv, d] with heads and d contiguous")
    with torch.cuda.device(dev):
        L.call("llmqrt_kv_append", L.ptr(k_cache), L.ptr(v_cache), k_cache.stride(0), k_cache.stride(1),
               L.ptr(k.contiguous()), L.ptr(v.contiguous()), L.ptr(cache_seqlens), int(start_pos),
               L.dtype_code(k_cache.dtype), B, S_new, Hkv, d, k_cache.shape[1], L.stream(dev))


def _rows_view(t, B, H, d, what):
    """Batch stride of a [B, H, d] tensor whose heads and d are contiguous (a slice of a fused row)."""
    if t.shape != (B, H, d) or t.stride(2) != 1 or t.stride(1) != d or t.data_ptr() % 16 or \
            (B > 1 and (t.stride(0) < H * d or t.stride(0) % 8)):
        raise RuntimeError(f"attn_decode: {what} must be [B, H, d] with heads and d contiguous, 16-byte aligned")
    return t.stride(0) if B > 1 else H * d


def attn_decode(q, k_cache, v_cache, seqlens, max_seqlen: int, softcap: float = 0.0, quantize: bool = False,
                k_new=None, v_new=None, cos=None, sin=None):
    """q [B, Hq, d] attends to rows [0, seqlens[b]) of the caches [Bc, Smax, Hkv, d]; returns [B, Hq, d].

    q may be a slice of a fused projection output (any batch stride, heads and d contiguous).
    quantize=True returns (out, out_q int8 [B, Hq*d], scale fp32 [B]): the per-token int8
    quantization of out, computed by the kernel that merges the KV splits.
    k_new / v_new [B, Hkv, d] (slices of a fused row allowed): the newest token's key and value are
    written into cache row seqlens[b] - 1 by the attention kernel itself; cos / sin (fp32
    [rows, d/2], see glue.rope_tables): q and the new key are rotated at that row's angle first.
    """
    dev = L.require_cuda(q, k_cache, v_cache, seqlens, k_new, v_new, cos, sin)
    B, Hq, d = q.shape
    Hkv = k_cache.shape[2]
    if k_cache.stride(3) != 1 or k_cache.stride(2) != d or v_cache.stride() != k_cache.stride():
        raise RuntimeError("attn_decode: caches must be [B, S, Hkv, d] with heads and d contiguous")
    if k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise TypeError("attn_decode: q and the caches must share one dtype")
    if seqlens.dtype != torch.int32:
        raise TypeError("attn_decode: seqlens must be int32")
    if B > 0 and (q.stride(2) != 1 or q.stride(1) != d or (B > 1 and (q.stride(0) < Hq * d or q.stride(0) % 8))
                  or q.data_ptr() % 16):
        q = q.contiguous()
    out = torch.empty((B, Hq, d), dtype=q.dtype, device=dev)
    out_q = torch.empty((B, Hq * d), dtype=torch.int8, device=dev) if quantize else None
    scale = torch.empty((B,), dtype=torch.float32, device=dev) if quantize else None
    q_stride = q.stride(0) if B > 1 else Hq * d
    fused = k_new is not None or cos is not None
    kv_stride = 0
    if k_new is not None:
        if v_new is None or k_new.dtype != q.dtype or v_new.dtype != q.dtype:
            raise RuntimeError("attn_decode: k_new and v_new go together, in q's dtype")
        kv_stride = _rows_view(k_new, B, Hkv, d, "k_new")
        if _rows_view(v_new, B, Hkv, d, "v_new") != kv_stride:
            raise RuntimeError("attn_decode: k_new and v_new must share one batch stride")
    if cos is not None:
        if sin is None or cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.shape != sin.shape or \
                cos.shape[-1] != d // 2 or not cos.is_contiguous() or not sin.is_contiguous():
            raise RuntimeError("attn_decode: cos / sin must be contiguous fp32 [rows, d/2]")
    with torch.cuda.device(dev):
        if fused:
            L.call("llmqrt_attn_decode_append", L.ptr(q), q_stride, L.ptr(k_new), L.ptr(v_new), kv_stride, L.ptr(cos),
                   L.ptr(sin), cos.shape[0] if cos is not None else 0, L.ptr(k_cache), L.ptr(v_cache),
                   k_cache.stride(0), k_cache.stride(1), L.ptr(seqlens), L.ptr(out), L.ptr(out_q), L.ptr(scale),
                   L.dtype_code(q.dtype), B, Hq, Hkv, d, int(max_seqlen), float(softcap), L.ptr(L.workspace(dev)),
                   L.stream(dev))
        else:
            L.call("llmqrt_attn_decode", L.ptr(q), q_stride, L.ptr(k_cache), L.ptr(v_cache), k_cache.stride(0),
                   k_cache.stride(1), L.ptr(seqlens), L.ptr(out), L.ptr(out_q), L.ptr(scale), L.dtype_code(q.dtype), B,
                   Hq, Hkv, d, int(max_seqlen), float(softcap), L.ptr(L.workspace(dev)), L.stream(dev))
    return (out, out_q, scale) if quantize else out


def flash_attn_with_kvcache(q, k_cache, v_cache, k=None, v=None, rotary_cos=None, rotary_sin=None,
                            cache_seqlens=None, cache_batch_idx=None, block_table=None, softmax_scale=None,
                            causal=False, window_size=(-1, -1), softcap=0.0, rotary_interleaved=True,
                            alibi_slopes=None, num_splits=0, max_seqlen_k=None):
    """Decode step over the KV cache.

    If k / v are given they are first written in place into the caches at row cache_seqlens[b];
    attention then covers rows [0, cache_seqlens[b] + k.shape[1]).  q is [B, 1, Hq, d] (one new token per
    sequence); the causal flag is immaterial for a single query.  `max_seqlen_k` (an addition to the
    flash-attn signature) bounds the longest sequence after the append so that the split-KV grid can be
    sized without reading cache_seqlens back; it defaults to the cache capacity.
    rotary_cos / rotary_sin ([rows, d/2], with k and v of one token and rotary_interleaved=False): q and
    the new key are rotated at angle row cache_seqlens[b] inside the attention kernel (half-split
    pairing, the convention of the reference's RoPE module); the interleaved pairing is not offered.
    """
    _check_common(q, softmax_scale, 0.0, window_size, alibi_slopes)
    if cache_batch_idx is not None or block_table is not None:
        raise NotImplementedError("llmqrt_b200 attention: batch indirection and paged caches are not supported")
    rotary = rotary_cos is not None or rotary_sin is not None
    if rotary and (rotary_interleaved or k is None or k.shape[1] != 1 or rotary_cos is None or rotary_sin is None):
        raise NotImplementedError("llmqrt_b200 attention: in-kernel rotary needs rotary_interleaved=False, both "
                                  "tables, and k / v of exactly one new token")
    B, Sq, Hq, d = q.shape
    if Sq != 1:
        raise NotImplementedError("flash_attn_with_kvcache: one query token per sequence (use flash_attn_func for prefill)")
    dev = L.require_cuda(q, k_cache, v_cache, k, v)
    if cache_seqlens is None:
        raise RuntimeError("flash_attn_with_kvcache: cache_seqlens is required")
    if isinstance(cache_seqlens, int):
        cache_seqlens = torch.full((B,), cache_seqlens, dtype=torch.int32, device=dev)
    seqlens = cache_seqlens
    cap = k_cache.shape[1]
    bound = min(cap, max_seqlen_k) if max_seqlen_k is not None else cap
    if k is not None:
        if v is None:
            raise RuntimeError("flash_attn_with_kvcache: k and v must be given together")
        seqlens = cache_seqlens + k.shape[1]
        if rotary:
            Hkv = k_cache.shape[2]
            out = attn_decode(q.reshape(B, Hq, d), k_cache, v_cache, seqlens, bound, softcap,
                              k_new=k.to(k_cache.dtype).reshape(B, Hkv, d).contiguous(),
                              v_new=v.to(v_cache.dtype).reshape(B, Hkv, d).contiguous(),
                              cos=rotary_cos.float().contiguous(), sin=rotary_sin.float().contiguous())
            return out.reshape(B, 1, Hq, d)
        kv_append(k_cache, v_cache, k.to(k_cache.dtype), v.to(v_cache.dtype), cache_seqlens=cache_seqlens)
    out = attn_decode(q.reshape(B, Hq, d), k_cache, v_cache, seqlens, bound, softcap)
    return out.reshape(B, 1, Hq, d)

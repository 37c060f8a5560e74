"""GQA attention over the KV cache, RoPE, RMSNorm (test oracle; see oracle/__init__.py).

The reference calls the third-party flash-attn package
(runtime/nn_models/modules/nonlinear/attn.py:10-15, 290-315) and has no test
or stored vector for it.  The functions below restate that package's
documented operator semantics in fp32/fp64; tests/test_gpu_attention_pin.py
pins them against the installed package on the GPU.
"""
from __future__ import annotations

import math

import torch


def _softcap(s: torch.Tensor, softcap: float) -> torch.Tensor:
    return s if softcap == 0.0 else softcap * torch.tanh(s / softcap)


def attention_prefill(q, k, v, causal: bool = True, softcap: float = 0.0) -> torch.Tensor:
    """O = softmax(Q K^T / sqrt(d)) V over the new tokens, call site attn.py:290-298.

    q [B,S,Hq,d], k/v [B,Sk,Hkv,d]; query head h reads kv head h // (Hq/Hkv);
    the causal mask is aligned to the end of the key sequence (query i sees
    keys j <= i + Sk - S).  Returns [B,S,Hq,d] in q's dtype.
    """
    B, S, Hq, d = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    rep = Hq // Hkv
    qf = q.to(torch.float64).permute(0, 2, 1, 3)                       # B,Hq,S,d
    kf = k.to(torch.float64).permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.to(torch.float64).permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = _softcap(qf @ kf.transpose(-1, -2) / math.sqrt(d), softcap)
    if causal:
        i = torch.arange(S).reshape(-1, 1)
        j = torch.arange(Sk).reshape(1, -1)
        s = s.masked_fill(j > i + (Sk - S), float("-inf"))
    p = torch.softmax(s, dim=-1)
    return (p @ vf).permute(0, 2, 1, 3).to(q.dtype)


def attention_decode_kvcache(q, k_cache, v_cache, k, v, cache_seqlens, softcap: float = 0.0):
    """flash_attn_with_kvcache semantics, call site attn.py:300-315.

    If k/v are given they are first written IN PLACE into the caches at row
    cache_seqlens[b]; attention then covers rows [0, cache_seqlens[b] + S_new).
    q [B,1,Hq,d], caches [Bc, Smax, Hkv, d], k/v [B,1,Hkv,d] or None,
    cache_seqlens int32 [B].  Returns [B,1,Hq,d].
    """
    B, Sq, Hq, d = q.shape
    outs = []
    for b in range(B):
        L = int(cache_seqlens[b])
        if k is not None:
            n_new = k.shape[1]
            k_cache[b, L:L + n_new] = k[b].to(k_cache.dtype)
            v_cache[b, L:L + n_new] = v[b].to(v_cache.dtype)
            L += n_new
        outs.append(attention_prefill(q[b:b + 1], k_cache[b:b + 1, :L], v_cache[b:b + 1, :L],
                                      causal=True, softcap=softcap))
    return torch.cat(outs, dim=0)


def rope_table(head_dim: int, max_seq_len: int, theta: float) -> torch.Tensor:
    """Angles[pos, i] = pos * theta**(-2i/d), fp32, as precompute_freqs_cis (attn.py:37-43)."""
    freqs = 1.0 / (theta ** (torch.arange(0, head_dim, 2)[: head_dim // 2].float() / head_dim))
    return torch.outer(torch.arange(max_seq_len), freqs).float()


def rope_apply(x: torch.Tensor, start_pos: int, theta: float, max_seq_len: int) -> torch.Tensor:
    """Rotary embedding with half-split pairing (element i pairs with i + d/2).

    Follows RoPE.forward, attn.py:53-87: fp32 complex multiply of
    (x[i] + j x[i+d/2]) by exp(j * angle[pos, i]) with positions
    start_pos .. start_pos+S-1 shared by the batch; result cast to x's dtype.
    x: [B, S, H, d].
    """
    B, S, H, d = x.shape
    ang = rope_table(d, max_seq_len, theta)[start_pos:start_pos + S]          # [S, d/2]
    cos, sin = torch.cos(ang), torch.sin(ang)
    cos = cos.reshape(1, S, 1, d // 2)
    sin = sin.reshape(1, S, 1, d // 2)
    xf = x.to(torch.float32)
    a, b = xf[..., : d // 2], xf[..., d // 2:]
    return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1).to(x.dtype)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """weight * T(x32 * rsqrt(mean(x32^2) + eps)), runtime/nn_models/modules/nonlinear/norm.py:10-16."""
    x32 = x.to(torch.float32)
    inv = torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + eps)
    return weight * (x32 * inv).to(x.dtype)


def cache_update(k_cache, v_cache, xk, xv, start_pos: int):
    """cache[:B, start:start+S] = x, runtime/nn_models/modules/nonlinear/cache.py:41-46."""
    B, S = xk.shape[0], xk.shape[1]
    k_cache[:B, start_pos:start_pos + S] = xk.to(k_cache.dtype)
    v_cache[:B, start_pos:start_pos + S] = xv.to(v_cache.dtype)

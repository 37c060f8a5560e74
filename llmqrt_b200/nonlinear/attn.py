"""Fused attention block with the reference's interface
(QuantAttentionFused, runtime/nn_models/modules/nonlinear/attn.py:129-338).

Same constructor arguments, attributes (`start_pos`, `cache`, `cache_batch_size`, ...) and return
triple.  Data flow per call: projections -> rotary embedding fused with the KV-cache write -> prefill
attention over the new tokens (seqlen > 1) or decode attention over the cache (seqlen == 1) -> o_proj.

The reference's decode branch writes the new K/V at `start_pos` and then lets the attention op append
the same K/V again at `start_pos + 1` (attn.py:275-303), so the newest token is attended twice.  That
is reproduced when REFERENCE_DOUBLE_APPEND is True (default, for drop-in parity); set it to False for
the plain "each token once" behaviour.
"""
from __future__ import annotations

import os

import torch
import torch.nn as nn

from .. import attention, glue
from .cache import WindowedCache


class RoPE(nn.Module):
    """Half-split rotary embedding (ref attn.py:27-87); tables built like precompute_freqs_cis."""

    def __init__(self, head_dim, max_seq_len, device, rope_theta):
        super().__init__()
        self.head_dim = head_dim
        self.cos, self.sin = glue.rope_tables(head_dim, max_seq_len, rope_theta, device)

    def forward(self, xq, xk, start_pos: int, seqlen: int, partial: bool = False):
        if partial:
            raise NotImplementedError("partial rotary embedding is not supported")
        xq, xk = xq.contiguous(), xk.contiguous()
        glue.rope_kv_write(xq, xk, None, self.cos, self.sin, pos0=start_pos)
        return xq, xk


class QuantAttentionFused(nn.Module):
    REFERENCE_DOUBLE_APPEND = True

    def __init__(self, hidden_size, n_heads, n_kv_heads, qkv_layer, o_proj, dev, q_proj=None, k_proj=None,
                 v_proj=None, max_seq_len=2048, use_alibi=False, attention_shapes=None, rope_theta=10000,
                 partial_rotary_factor=1.0, head_dim=None, attn_logit_softcapping=0.0, q_norm=None, k_norm=None,
                 **kwargs):
        super().__init__()
        if use_alibi:
            raise NotImplementedError("ALiBi is not supported (the reference never applies it either)")
        if partial_rotary_factor != 1.0:
            raise NotImplementedError("partial rotary embedding is not supported")
        self.hidden_size, self.n_heads, self.n_kv_heads = hidden_size, n_heads, n_kv_heads
        self.n_kv_groups = n_heads // n_kv_heads if n_kv_heads != 0 else 0
        self.head_dim = head_dim if head_dim is not None else hidden_size // n_heads
        self.qkv_proj, self.q_proj, self.k_proj, self.v_proj, self.o_proj = qkv_layer, q_proj, k_proj, v_proj, o_proj
        self.q_norm, self.k_norm = q_norm, k_norm
        self.start_pos = 0
        self.use_alibi = False
        self.cache_batch_size = int(os.getenv("AWQ_BATCH_SIZE", "1"))
        if kwargs.get("max_length") is not None:
            max_seq_len = kwargs["max_length"]
        self.max_seq_len = max_seq_len
        self.is_hf_transformers = False
        self.rope_theta = rope_theta
        self.cache = WindowedCache(self.cache_batch_size, n_heads, n_kv_heads, self.head_dim, max_seq_len, dev)
        self.rotary_dim = self.head_dim
        self.rope = RoPE(self.head_dim, max_seq_len, dev, rope_theta)
        self.is_neox = kwargs.get("is_neox", True)
        self.attn_logit_softcapping = attn_logit_softcapping

    @torch.no_grad()
    def forward(self, hidden_states: torch.Tensor, *args, **kwargs):
        bsz, seqlen, _ = hidden_states.shape
        if bsz != self.cache_batch_size:
            if bsz > self.cache_batch_size:
                self.cache.increase_batch_size(bsz)
            else:
                self.cache.decrease_batch_size(bsz)
            self.cache_batch_size = bsz
            self.start_pos = 0

        H, Hkv, d = self.n_heads, self.n_kv_heads if self.n_kv_heads else self.n_heads, self.head_dim
        if self.q_proj is not None:
            xq = self.q_proj(hidden_states).view(bsz, seqlen, H, d)
            xk = self.k_proj(hidden_states).view(bsz, seqlen, Hkv, d)
            xv = self.v_proj(hidden_states).view(bsz, seqlen, Hkv, d)
        else:
            xqkv = self.qkv_proj(hidden_states).view(bsz, seqlen, H + 2 * Hkv, d)
            xq, xk, xv = xqkv[:, :, :H], xqkv[:, :, H:H + Hkv], xqkv[:, :, H + Hkv:]
        if self.q_norm is not None:
            xq = self.q_norm(xq)
        if self.k_norm is not None:
            xk = self.k_norm(xk)

        self.cache.to(xq)
        xq, xk, xv = xq.contiguous(), xk.contiguous(), xv.contiguous()
        # rotary embedding of q and k, and cache[:, start_pos : start_pos + seqlen] = (k, v), one kernel
        glue.rope_kv_write(xq, xk, xv, self.rope.cos, self.rope.sin, pos0=self.start_pos,
                           k_cache=self.cache.k[:bsz], v_cache=self.cache.v[:bsz])
        if seqlen > 1:
            output = attention.flash_attn_func(q=xq, k=xk, v=xv, causal=True, softcap=self.attn_logit_softcapping)
        else:
            cap = self.cache.k.shape[1]
            if self.REFERENCE_DOUBLE_APPEND and self.start_pos + 1 < cap:
                seqlens = torch.full((bsz,), self.start_pos + 1, dtype=torch.int32, device=xq.device)
                output = attention.flash_attn_with_kvcache(
                    q=xq, k=xk, k_cache=self.cache.k, v=xv, v_cache=self.cache.v, cache_seqlens=seqlens,
                    causal=True, softcap=self.attn_logit_softcapping, max_seqlen_k=self.start_pos + 2)
            else:
                seqlens = torch.full((bsz,), self.start_pos + 1, dtype=torch.int32, device=xq.device)
                output = attention.flash_attn_with_kvcache(
                    q=xq, k_cache=self.cache.k, v_cache=self.cache.v, cache_seqlens=seqlens, causal=True,
                    softcap=self.attn_logit_softcapping, max_seqlen_k=self.start_pos + 1)
        attention_weight = output.reshape(bsz, seqlen, -1)
        attn_output = self.o_proj(attention_weight)
        self.start_pos += seqlen
        if self.is_hf_transformers and not kwargs.get("use_cache", False):
            self.start_pos = 0
        past_key_value = [torch.zeros(1, 1, self.start_pos, 1)]
        return attn_output, attention_weight, past_key_value

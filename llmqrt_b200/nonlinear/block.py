"""Pre-norm decoder block and layer stack with the reference's interfaces
(runtime/nn_models/modules/nonlinear/block.py:8-78, model.py:11-62)."""
from __future__ import annotations

from typing import List

import torch
import torch.nn as nn

from .attn import QuantAttentionFused


class LlamaLikeBlock(nn.Module):
    def __init__(self, hidden_size, n_heads, n_kv_heads, qkv_layer, q_proj, k_proj, v_proj, o_proj, mlp, norm_1,
                 norm_2, dev, max_seq_len, rope_theta=10000, partial_rotary_factor=1.0, use_alibi=False,
                 head_dim=None):
        super().__init__()
        self.n_heads, self.n_kv_heads = n_heads, n_kv_heads
        self.head_dim = head_dim if head_dim else hidden_size // n_heads
        self.hidden_size = hidden_size
        self.norm_1 = norm_1.to(dev)
        self.attn = QuantAttentionFused(hidden_size, n_heads, n_kv_heads, qkv_layer, o_proj, dev=dev, q_proj=q_proj,
                                        k_proj=k_proj, v_proj=v_proj, max_seq_len=max_seq_len, use_alibi=use_alibi,
                                        rope_theta=rope_theta, partial_rotary_factor=partial_rotary_factor,
                                        head_dim=head_dim).to(dev)
        self.norm_2 = norm_2.to(dev)
        self.mlp = mlp.to(dev)
        self.device = dev

    def forward(self, hidden_states):
        attn_output, _, _ = self.attn.forward(hidden_states=self.norm_1(hidden_states))
        h = hidden_states.to(attn_output.device) + attn_output
        return h + self.mlp.forward(self.norm_2(h))


class LlamaLikeModel(nn.Module):
    def __init__(self, vocab_size, blocks, embedding, norm):
        super().__init__()
        self.vocab_size = vocab_size
        self.embedding = embedding
        self.blocks: List[LlamaLikeBlock] = nn.ModuleList(blocks)
        self.norm = norm
        self.last_forward_num_tokens = 0

    @property
    def embed_tokens(self):
        return self.embedding

    @property
    def layers(self):
        return self.blocks

    @torch.inference_mode()
    def forward(self, input_ids: torch.Tensor, *args, **kwargs):
        # keep only the new tokens once the context has been processed (ref fused_utils.py:28-40)
        n_in = input_ids.shape[-1]
        n_new = n_in
        if n_in != 1:
            n_new = n_in - self.last_forward_num_tokens
            if n_new == 1:
                input_ids = input_ids[:, -1:]
        self.last_forward_num_tokens += n_new
        seqlen = input_ids.shape[1]
        for block in self.blocks:            # reset / roll the caches (ref fused_utils.py:12-25)
            a = block.attn
            exceeded = a.start_pos + seqlen > a.max_seq_len
            if seqlen > 1 and (exceeded or a.start_pos > 0):
                a.start_pos = a.cache.roll_kv_n_steps(a.start_pos, n=a.start_pos)
            elif seqlen == 1 and exceeded:
                a.start_pos = a.cache.roll_kv_n_steps(a.start_pos, n=100)
        h = self.embedding(input_ids)
        for layer in self.blocks:
            h = layer(h.to(layer.device))
        return self.norm(h)

"""CPU restatement of the int8 W8A8 Qwen2 decoder step (test oracle; see oracle/__init__.py).

Follows the reference's fused model flow -- LlamaLikeModel.forward
(runtime/nn_models/modules/nonlinear/model.py:33-62), LlamaLikeBlock.forward (block.py:64-78),
QuantAttentionFused.forward (attn.py:212-338) and the Hugging Face Qwen2MLP it keeps -- with every
linear layer computed as  per-token int8 quantize -> exact int32 GEMM -> per-token x per-channel
dequantize (+ bias)  from the other oracle modules.  Tensor parallelism is emulated by looping over
the ranks' weight shards and summing the row-parallel partial outputs in the 16-bit dtype, in rank
order.
"""
from __future__ import annotations

import torch

from . import attention as oattn
from . import gemm as ogemm
from . import quant as oquant


def _linear(x, w_q, w_s, bias, dt):
    xq, xs = oquant.quantize_int8(x, per_token=True)
    return ogemm.int8_linear_per_channel(xq, w_q, bias, xs.float(), w_s, dt)


class Qwen2Oracle:
    """`shards` is a list (one entry per tensor-parallel rank) of dicts of CPU tensors with the keys
    used below; `cfg` needs hidden, head_dim, rms_eps, rope_theta, dtype."""

    def __init__(self, cfg, shards, batch, max_seq_len):
        self.cfg, self.shards, self.S = cfg, shards, max_seq_len
        self.caches = [[(torch.zeros(batch, max_seq_len, s["hkv"], cfg.head_dim, dtype=cfg.dtype),
                         torch.zeros(batch, max_seq_len, s["hkv"], cfg.head_dim, dtype=cfg.dtype))
                        for _ in s["layers"]] for s in shards]
        self.pos = 0

    def _sum_partials(self, parts):
        out = parts[0]
        for p in parts[1:]:
            out = out + p                       # 16-bit adds, rank order (what an allreduce of 16-bit data does)
        return out

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [B, S] at positions pos..pos+S-1 -> logits [B, vocab] of the last position."""
        cfg, d, dt = self.cfg, self.cfg.head_dim, self.cfg.dtype
        B, S = tokens.shape
        s0 = self.shards[0]
        h = s0["embed"][tokens.reshape(-1)]
        n_layers = len(s0["layers"])
        for li in range(n_layers):
            x = oattn.rmsnorm(h, s0["layers"][li]["ln1"], cfg.rms_eps)
            parts = []
            for r, sh in enumerate(self.shards):
                L = sh["layers"][li]
                hq, hkv = sh["hq"], sh["hkv"]
                qkv = _linear(x, L["wqkv"], L["sqkv"], L["bqkv"], dt).view(B, S, hq + 2 * hkv, d)
                q, k, v = qkv[:, :, :hq], qkv[:, :, hq:hq + hkv], qkv[:, :, hq + hkv:]
                q = oattn.rope_apply(q, self.pos, cfg.rope_theta, self.S)
                k = oattn.rope_apply(k, self.pos, cfg.rope_theta, self.S)
                kc, vc = self.caches[r][li]
                oattn.cache_update(kc, vc, k, v, self.pos)
                L_tot = self.pos + S
                a = oattn.attention_prefill(q, kc[:, :L_tot], vc[:, :L_tot], causal=True)
                parts.append(_linear(a.reshape(B * S, hq * d), L["wo"], L["so"], None, dt))
            h = h + self._sum_partials(parts)
            y = oattn.rmsnorm(h, s0["layers"][li]["ln2"], cfg.rms_eps)
            parts = []
            for sh in self.shards:
                L = sh["layers"][li]
                gu = _linear(y, L["wgu"], L["sgu"], None, dt)
                I = gu.shape[1] // 2
                m = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
                parts.append(_linear(m, L["wd"], L["sd"], None, dt))
            h = h + self._sum_partials(parts)
        self.pos += S
        y = oattn.rmsnorm(h.view(B, S, -1)[:, -1], s0["norm_f"], cfg.rms_eps)
        logits = [(y.double() @ sh["lm_head"].double().t()).to(dt) for sh in self.shards]
        return torch.cat(logits, dim=1)

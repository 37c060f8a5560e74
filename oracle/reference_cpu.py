"""The reference's own CPU-runnable path for the quantized linears, for timing (test / benchmark
infrastructure; see oracle/__init__.py).

The reference has no CPU kernels; what runs on a CPU is its torch "dequantize, then matmul" code:
  * int8: `linear(xq.to(T) * input_scale, wq.to(T) * weight_scale, bias)`, the ground truth of
    runtime/unittest/test_sq_linear.py:16-25 and the commented "naive impl" of
    runtime/nn_models/modules/linear/linear_sq.py:118-125;
  * fp8: the fallback branch of fp8_gemm, runtime/nn_models/modules/linear/linear_fp8.py:97-101;
  * AWQ: dequantize_gemm + matmul, runtime/nn_models/modules/linear/linear_awq.py:64-65.
Attention has no CPU implementation in the reference (it calls flash-attn); the decode-attention
sample below is a plain torch restatement and is labelled as such by the benchmark.
"""
from __future__ import annotations

import time

import torch

from . import awq as oawq


def sq_linear(xq, x_scale, wq, w_scale, bias, dtype):
    return torch.nn.functional.linear(xq.to(dtype) * x_scale.to(dtype), wq.to(dtype) * w_scale.to(dtype), bias)


def fp8_linear(xq, x_scale, wq, w_scale, bias, dtype):
    return torch.nn.functional.linear(xq.to(dtype) * x_scale.to(dtype), wq.to(dtype) * w_scale.to(dtype), bias)


def awq_linear(x, qweight, qzeros, scales, group_size):
    return torch.matmul(x, oawq.dequantize(qweight, qzeros, scales, group_size))


def decode_attention(q, k_cache, v_cache, ctx):
    """q [B,Hq,d] over the first `ctx` rows of caches [B,S,Hkv,d]; GQA by repeat, fp32 softmax."""
    B, Hq, d = q.shape
    rep = Hq // k_cache.shape[2]
    k = k_cache[:, :ctx].permute(0, 2, 1, 3).repeat_interleave(rep, dim=1).float()
    v = v_cache[:, :ctx].permute(0, 2, 1, 3).repeat_interleave(rep, dim=1).float()
    s = torch.einsum("bhd,bhkd->bhk", q.float(), k) * d ** -0.5
    return torch.einsum("bhk,bhkd->bhd", torch.softmax(s, dim=-1), v).to(q.dtype)


class Qwen2LayerSample:
    """One random-init decoder layer's quantized linears (q, k, v, o, gate, up, down as seven separate
    layers, as the reference keeps them for SmoothQuant) plus decode attention, on the CPU."""

    def __init__(self, hidden, inter, hq, hkv, d, batch, ctx, dtype=torch.bfloat16, seed=0):
        g = torch.Generator().manual_seed(seed)
        self.dtype, self.batch, self.ctx, self.hq, self.hkv, self.d = dtype, batch, ctx, hq, hkv, d
        shapes = {"q": (hq * d, hidden), "k": (hkv * d, hidden), "v": (hkv * d, hidden), "o": (hidden, hq * d),
                  "gate": (inter, hidden), "up": (inter, hidden), "down": (hidden, inter)}
        self.w = {n: (torch.randint(-127, 128, s, generator=g, dtype=torch.int8), torch.rand(s[0], 1, generator=g) * 1e-3)
                  for n, s in shapes.items()}
        self.x = {n: (torch.randint(-127, 128, (batch, s[1]), generator=g, dtype=torch.int8),
                      torch.rand(batch, 1, generator=g) * 1e-2) for n, s in shapes.items()}
        self.kc = torch.randn(batch, ctx, hkv, d, generator=g).to(dtype)
        self.vc = torch.randn(batch, ctx, hkv, d, generator=g).to(dtype)
        self.qv = torch.randn(batch, hq, d, generator=g).to(dtype)

    def step(self) -> float:
        """Runs the layer once; returns seconds."""
        t0 = time.perf_counter()
        for n, (wq, ws) in self.w.items():
            xq, xs = self.x[n]
            sq_linear(xq, xs, wq, ws, None, self.dtype)
        decode_attention(self.qv, self.kc, self.vc, self.ctx)
        return time.perf_counter() - t0


def time_lm_head(hidden, vocab, batch, dtype=torch.bfloat16, seed=0) -> float:
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(vocab, hidden, generator=g).to(dtype)
    x = torch.randn(batch, hidden, generator=g).to(dtype)
    torch.nn.functional.linear(x, w)
    t0 = time.perf_counter()
    torch.nn.functional.linear(x, w)
    return time.perf_counter() - t0

"""Random-init Qwen2 decoder running entirely on this package's kernels (SmoothQuant-style int8 W8A8,
per-token activation scales x per-output-channel weight scales), with Megatron tensor parallelism.

This is the harness behind the end-to-end decode benchmark.  It follows the data flow of the
reference's fused model (runtime/nn_models/modules/nonlinear/model.py:33-62, block.py:64-78,
attn.py:212-338) with the per-op torch chains replaced by fused kernels:

    RMSNorm+quant -> qkv GEMM(+bias) -> RoPE+KV write -> attention -> quant -> o_proj GEMM -> [allreduce]
    -> residual+RMSNorm+quant -> gate_up GEMM -> SiLU*up+quant -> down GEMM -> [allreduce]

Tensor parallelism: q/k/v, gate and up are column-parallel (by heads / output channels), o_proj and
down_proj row-parallel (each rank quantizes its own activation slice with its own per-token scale, the
16-bit partial outputs are summed by an allreduce).  KV heads that cannot be divided among the ranks
are replicated and their query heads split (28/4 heads on 8 ranks: 4 + 3 query heads per KV head).
The lm_head is column-parallel over the vocabulary; greedy sampling reduces (max, argmax) pairs.
"""
from __future__ import annotations

import dataclasses
import os
from typing import Optional

import torch

from . import attention, glue, ops
from .tp import PeerAllreduce, allreduce_sum, greedy_select, head_assignment, rows_of_heads


@dataclasses.dataclass
class Qwen2Config:
    num_layers: int = 28
    hidden: int = 3584
    intermediate: int = 18944
    num_heads: int = 28
    num_kv_heads: int = 4
    head_dim: int = 128
    vocab: int = 152064
    rms_eps: float = 1e-6
    rope_theta: float = 1e6
    dtype: torch.dtype = torch.bfloat16

    @staticmethod
    def qwen2_7b() -> "Qwen2Config":
        return Qwen2Config()

    @staticmethod
    def tiny() -> "Qwen2Config":
        return Qwen2Config(num_layers=2, hidden=256, intermediate=512, num_heads=4, num_kv_heads=2, head_dim=64,
                           vocab=1024)


def _randn_rows(rows: int, cols: int, seed: int, std: float, device, dtype) -> torch.Tensor:
    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(rows, cols, generator=g, device=device, dtype=torch.float32) * std).to(dtype)


def _quantize_weight(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Symmetric int8 per output channel (absmax / 127), the recipe of
    runtime/utils/quantization_utils.py:28-38; set-up code, runs once."""
    w32 = w.float()
    scale = (w32.abs().amax(dim=1, keepdim=True) / 127).clamp_min(1e-8)
    q = torch.round(w32 / scale).clamp(-128, 127).to(torch.int8)
    return q.contiguous(), scale.reshape(-1).contiguous()


class _Layer:
    __slots__ = ("ln1", "ln2", "wqkv", "sqkv", "bqkv", "wo", "so", "wgu", "sgu", "wd", "sd", "k_cache", "v_cache")


class Qwen2Decoder:
    """One tensor-parallel rank of the model.  `group` is a torch.distributed process group (or None)."""

    def __init__(self, cfg: Qwen2Config, device, batch: int, max_seq_len: int, tp: int = 1, rank: int = 0,
                 group=None, seed: int = 0):
        self.cfg, self.device, self.tp, self.rank, self.group = cfg, torch.device(device), tp, rank, group
        self.batch, self.max_seq_len = batch, max_seq_len
        d, dt, dev = cfg.head_dim, cfg.dtype, self.device
        # Decode-sized partial sums go over peer-mapped buffers (LLMQRT_ALLREDUCE=nccl keeps NCCL for
        # everything); prefill-sized ones always use NCCL.
        self.comm = None
        if tp > 1 and os.environ.get("LLMQRT_ALLREDUCE", "peer") != "nccl":
            self.comm = PeerAllreduce(self.device, rank, tp, max(batch, 8) * cfg.hidden * 2, group)
        self.q_heads, self.kv_heads = head_assignment(cfg.num_heads, cfg.num_kv_heads, tp, rank)
        self.hq, self.hkv = len(self.q_heads), len(self.kv_heads)
        if cfg.intermediate % tp or (cfg.intermediate // tp) % 16:
            raise ValueError("intermediate size must split into multiples of 16 per rank")
        if cfg.vocab % tp:
            raise ValueError("vocabulary must divide among the ranks")
        self.inter_local = cfg.intermediate // tp
        i0 = rank * self.inter_local
        q_rows = torch.tensor(rows_of_heads(self.q_heads, d), device=dev)
        kv_rows = torch.tensor(rows_of_heads(self.kv_heads, d), device=dev)

        self.layers: list[_Layer] = []
        for li in range(cfg.num_layers):
            s = seed * 1000003 + li * 16
            L_ = _Layer()
            L_.ln1 = torch.ones(cfg.hidden, dtype=dt, device=dev)
            L_.ln2 = torch.ones(cfg.hidden, dtype=dt, device=dev)
            wq = _randn_rows(cfg.num_heads * d, cfg.hidden, s + 1, 0.02, dev, dt)[q_rows]
            wk = _randn_rows(cfg.num_kv_heads * d, cfg.hidden, s + 2, 0.02, dev, dt)[kv_rows]
            wv = _randn_rows(cfg.num_kv_heads * d, cfg.hidden, s + 3, 0.02, dev, dt)[kv_rows]
            L_.wqkv, L_.sqkv = _quantize_weight(torch.cat([wq, wk, wv], dim=0))
            bq = _randn_rows(1, cfg.num_heads * d, s + 4, 0.02, dev, dt)[0][q_rows]
            bk = _randn_rows(1, cfg.num_kv_heads * d, s + 5, 0.02, dev, dt)[0][kv_rows]
            bv = _randn_rows(1, cfg.num_kv_heads * d, s + 6, 0.02, dev, dt)[0][kv_rows]
            L_.bqkv = torch.cat([bq, bk, bv]).contiguous()
            del wq, wk, wv
            wo = _randn_rows(cfg.hidden, cfg.num_heads * d, s + 7, 0.02, dev, dt)[:, q_rows]
            L_.wo, L_.so = _quantize_weight(wo)
            del wo
            wg = _randn_rows(cfg.intermediate, cfg.hidden, s + 8, 0.02, dev, dt)[i0:i0 + self.inter_local]
            wu = _randn_rows(cfg.intermediate, cfg.hidden, s + 9, 0.02, dev, dt)[i0:i0 + self.inter_local]
            L_.wgu, L_.sgu = _quantize_weight(torch.cat([wg, wu], dim=0))
            del wg, wu
            wd = _randn_rows(cfg.hidden, cfg.intermediate, s + 10, 0.02, dev, dt)[:, i0:i0 + self.inter_local]
            L_.wd, L_.sd = _quantize_weight(wd)
            del wd
            L_.k_cache = torch.zeros(batch, max_seq_len, self.hkv, d, dtype=dt, device=dev)
            L_.v_cache = torch.zeros_like(L_.k_cache)
            self.layers.append(L_)

        self.embed = _randn_rows(cfg.vocab, cfg.hidden, seed * 1000003 + 900001, 0.02, dev, dt)
        self.norm_f = torch.ones(cfg.hidden, dtype=dt, device=dev)
        v_local = cfg.vocab // tp
        self.vocab0 = rank * v_local
        self.lm_head = _randn_rows(cfg.vocab, cfg.hidden, seed * 1000003 + 900002, 0.02, dev, dt)[
            self.vocab0:self.vocab0 + v_local].contiguous()
        self.cos, self.sin = glue.rope_tables(d, max_seq_len, cfg.rope_theta, dev)
        self.pos = 0                                                   # host copy of the position
        self.pos_dev = torch.zeros(1, dtype=torch.int32, device=dev)   # device copy read by the kernels
        self.seqlens = torch.zeros(batch, dtype=torch.int32, device=dev)
        self._graph = None
        self._graph_tokens = None
        self._graph_out = None

    # ------------------------------------------------------------------------------------------
    def export_shard(self) -> dict:
        """CPU copy of this rank's weights, in the form the CPU oracle of the decoder consumes."""
        keys = ("ln1", "ln2", "wqkv", "sqkv", "bqkv", "wo", "so", "wgu", "sgu", "wd", "sd")
        return {"hq": self.hq, "hkv": self.hkv, "embed": self.embed.cpu(), "norm_f": self.norm_f.cpu(),
                "lm_head": self.lm_head.cpu(),
                "layers": [{k: getattr(L_, k).cpu() for k in keys} for L_ in self.layers]}

    def weight_bytes(self) -> int:
        n = sum(t.numel() * t.element_size() for L_ in self.layers for t in (L_.wqkv, L_.wo, L_.wgu, L_.wd))
        return n + self.lm_head.numel() * self.lm_head.element_size()

    def _allreduce(self, x: torch.Tensor) -> torch.Tensor:
        return allreduce_sum(x, self.tp, self.group, self.comm)

    def _layers_forward(self, h: torch.Tensor, B: int, S: int, decode: bool, batch0: int = 0) -> torch.Tensor:
        """h [B*S, hidden] -> hidden state before the final norm.  decode: S == 1, positions from pos_dev."""
        cfg, d, dt = self.cfg, self.cfg.head_dim, self.cfg.dtype
        nq, nkv = self.hq * d, self.hkv * d
        pending = None                                                 # output of the previous MLP, not yet added
        for L_ in self.layers:
            # with a peer communicator the partial sums of the row-parallel projections are reduced
            # inside the RMSNorm kernel that consumes them; without one, by NCCL right after the GEMM
            _, h_new, xq, xs = glue.rmsnorm(h, L_.ln1, cfg.rms_eps, residual=pending, quantize=True, want_y=False,
                                            comm=self.comm)
            if h_new is not None:
                h = h_new
            qkv = ops.int8_linear_per_channel(xq, L_.wqkv, L_.bqkv, xs, L_.sqkv, dt, True)          # [M, nq + 2 nkv]
            qkv4 = qkv.view(B, S, self.hq + 2 * self.hkv, d)
            q, k, v = qkv4[:, :, :self.hq], qkv4[:, :, self.hq:self.hq + self.hkv], qkv4[:, :, self.hq + self.hkv:]
            kc, vc = L_.k_cache[batch0:batch0 + B], L_.v_cache[batch0:batch0 + B]
            if decode:
                # One kernel: q, k, v are read in place from the fused projection output, q and k are
                # rotated at the row's angle (seqlens == position + 1), k and v go into the cache,
                # and the kernel that finishes the attention also emits the per-token int8 row that
                # the output projection consumes.
                _, aq, a_s = attention.attn_decode(q[:, 0], kc, vc, self.seqlens[batch0:batch0 + B],
                                                   self.max_seq_len if self._capturing else self.pos + 1,
                                                   quantize=True, k_new=k[:, 0], v_new=v[:, 0],
                                                   cos=self.cos, sin=self.sin)
            else:
                glue.rope_kv_write(q, k, v, self.cos, self.sin, pos0=self.pos, pos_dev=None, k_cache=kc, v_cache=vc)
                attn = attention.flash_attn_func(q, k, v, causal=True)
                aq, _, a_s = ops.quantize_int8(attn.reshape(B * S, nq), per_token=True)
            M = B * S
            push = decode and self.comm is not None and self.comm.push_ok(M, cfg.hidden)
            if push:                                   # GEMM epilogue -> peers' buffers; the RMSNorm below gathers
                o = self.comm.linear_push(aq, L_.wo, None, a_s, L_.so, dt, True)
            else:
                o = ops.int8_linear_per_channel(aq, L_.wo, None, a_s, L_.so, dt, True)
            if self.comm is None:
                o = self._allreduce(o)
            _, h, yq, ys = glue.rmsnorm(h, L_.ln2, cfg.rms_eps, residual=o, quantize=True, want_y=False,
                                        comm=self.comm)
            gu = ops.int8_linear_per_channel(yq, L_.wgu, None, ys, L_.sgu, dt, True)                # [M, 2 I_local]
            _, mq, ms = glue.silu_mul(gu, quantize=True, want_y=False)
            if push:
                pending = self.comm.linear_push(mq, L_.wd, None, ms, L_.sd, dt, True)
            else:
                pending = ops.int8_linear_per_channel(mq, L_.wd, None, ms, L_.sd, dt, True)
            if self.comm is None:
                pending = self._allreduce(pending)
        return h, pending

    _capturing = False

    def _head(self, h: torch.Tensor, pending: torch.Tensor) -> torch.Tensor:
        """Final norm, vocabulary-parallel lm_head, greedy token per row."""
        y, _, _, _ = glue.rmsnorm(h, self.norm_f, self.cfg.rms_eps, residual=pending, comm=self.comm)
        logits = ops.gemm_16bit(y, self.lm_head)                                            # [M, V/tp]
        self.last_logits = logits
        val, idx = logits.max(dim=-1)
        return greedy_select(val, idx + self.vocab0, self.tp, self.group)

    # ------------------------------------------------------------------------------------------
    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor, chunk_sequences: int = 16) -> torch.Tensor:
        """tokens [B, S] (device, int64) at positions 0..S-1.  Returns the greedy next token per sequence [B]."""
        B, S = tokens.shape
        assert B == self.batch and S <= self.max_seq_len
        self.pos = 0
        out = []
        for b0 in range(0, B, chunk_sequences):
            b1 = min(B, b0 + chunk_sequences)
            h = self.embed[tokens[b0:b1].reshape(-1)]
            h, pending = self._layers_forward(h, b1 - b0, S, decode=False, batch0=b0)
            hl = h.view(b1 - b0, S, -1)[:, -1].contiguous()
            pl = pending.view(b1 - b0, S, -1)[:, -1].contiguous()
            out.append(self._head(hl, pl))
        self.pos = S
        self.pos_dev.fill_(S)
        self.seqlens.fill_(S + 1)          # rows [0, pos] are valid once the step's K/V are written
        return torch.cat(out)

    @torch.no_grad()
    def decode_step_host(self, tokens_in: torch.Tensor, tokens_out: torch.Tensor) -> None:
        """Serving-style step with HOST buffers: `tokens_in` / `tokens_out` are pinned CPU int64 [B] tensors.
        Copies the ids to the device, runs one decode step, copies the sampled ids back and waits for them."""
        dev_in = self._host_in if getattr(self, "_host_in", None) is not None else None
        if dev_in is None:
            dev_in = self._host_in = torch.empty(self.batch, dtype=torch.int64, device=self.device)
        dev_in.copy_(tokens_in, non_blocking=True)
        nxt = self.decode_step(dev_in, use_graph=True)
        tokens_out.copy_(nxt, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()

    def reset_position(self, pos: int) -> None:
        """Rewind (or advance) the decode position; cache rows at and beyond `pos` will be overwritten."""
        assert 0 <= pos < self.max_seq_len
        self.pos = pos
        self.pos_dev.fill_(pos)
        self.seqlens.fill_(pos + 1)

    def _decode_body(self, tokens: torch.Tensor) -> torch.Tensor:
        h = self.embed[tokens]
        h, pending = self._layers_forward(h, self.batch, 1, decode=True)
        nxt = self._head(h, pending)
        self.pos_dev += 1
        self.seqlens += 1
        return nxt

    @torch.no_grad()
    def decode_step(self, tokens: torch.Tensor, use_graph: bool = True) -> torch.Tensor:
        """One greedy decode step for the whole batch: tokens [B] (device) -> next tokens [B] (device).

        With use_graph the step is captured once into a CUDA graph (positions live on the device, so the
        same graph serves every step) and replayed; the returned tensor is then a static buffer that the
        next call overwrites.
        """
        if self.pos >= self.max_seq_len:
            raise RuntimeError("KV cache is full")
        if not use_graph:
            nxt = self._decode_body(tokens)
            self.pos += 1
            return nxt
        if self._graph is None:
            self._graph_tokens = tokens.clone()
            saved = (self.pos_dev.clone(), self.seqlens.clone())
            side = torch.cuda.Stream(self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):                              # warm-up outside capture
                self._decode_body(self._graph_tokens)
            torch.cuda.current_stream(self.device).wait_stream(side)
            torch.cuda.synchronize(self.device)
            self.pos_dev.copy_(saved[0])
            self.seqlens.copy_(saved[1])
            self._graph = torch.cuda.CUDAGraph()
            Qwen2Decoder._capturing = True
            try:
                with torch.cuda.graph(self._graph):
                    self._graph_out = self._decode_body(self._graph_tokens)
            finally:
                Qwen2Decoder._capturing = False
            self.pos_dev.copy_(saved[0])
            self.seqlens.copy_(saved[1])
        self._graph_tokens.copy_(tokens, non_blocking=True)
        self._graph.replay()
        self.pos += 1
        return self._graph_out

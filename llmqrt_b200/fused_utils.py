"""Fusion of projections that read the same input: q/k/v and gate/up.

Mirrors runtime/utils/fused_utils.py:43-123 (`fuse_qkv`, `fuse_linears`).  The reference fuses only AWQ
layers and returns SQ and FP8 layers unfused (fused_utils.py:47-56; FP8-dynamic fusion is left "as
homework", models/readme.md:6).  Here every scheme whose activation scale is computed from the input
at run time is fused -- the three projections then cost ONE activation quantization and ONE GEMM
launch:

    WQLinear_GEMM                         packed words / zeros / scales concatenated along N (as the reference)
    SqW8A8BBF16OBF16PerChannel            int8 rows, per-channel scales and bias concatenated (per-token activation scale)
    FP8DynamicLinear(per_tensor=False)    weight rows, per-channel scales and bias concatenated (per-token activation scale)

Schemes with ONE weight scale per tensor (SqW8A8BBF16OBF16PerTensor, FP8DynamicLinear(per_tensor=True))
and static activation scales (FP8StaticLinear) keep the reference's behaviour: q, k, v carry
different scales, the scalar-alpha kernels cannot express that, and the tuple is returned unchanged.

The concatenation is along output channels, so every output column is computed exactly as the
unfused layer would: the fused result is bit-identical to torch.cat of the three separate outputs.
"""
from __future__ import annotations

import torch

from .linear import FP8DynamicLinear, SqW8A8BBF16OBF16PerChannel, WQLinear_GEMM


def _cat_bias(layers):
    """Concatenated bias; layers without one contribute zeros.  None if no layer has a bias."""
    ref = next((l.bias for l in layers if l.bias is not None), None)
    if ref is None:
        return None
    return torch.cat([(l.bias.data if l.bias is not None
                       else torch.zeros(l.out_features, dtype=ref.dtype, device=ref.device)).to(ref.dtype)
                      for l in layers], dim=0)


def fusable(layer) -> bool:
    """Whether `layer`'s scheme allows projections of the same input to be fused."""
    if isinstance(layer, (WQLinear_GEMM, SqW8A8BBF16OBF16PerChannel)):
        return True
    return isinstance(layer, FP8DynamicLinear) and not layer.per_tensor


def fuse_linears(linears, device=None):
    """One layer computing torch.cat([l(x) for l in linears], dim=-1).  All layers must be of the same
    fusable class with equal in_features.  The inputs' buffers are released (like the reference,
    fused_utils.py:100-101, 119-120)."""
    first = linears[0]
    if not all(type(l) is type(first) and l.in_features == first.in_features for l in linears) or not fusable(first):
        raise TypeError("fuse_linears: layers must share one fusable class and in_features")
    out_features = sum(l.out_features for l in linears)
    has_bias = any(l.bias is not None for l in linears)
    if isinstance(first, WQLinear_GEMM):
        dev = device if device is not None else first.qweight.device
        fused = WQLinear_GEMM(first.w_bit, first.group_size, first.in_features, out_features, has_bias, dev)
        fused.qweight = torch.cat([l.qweight for l in linears], dim=1).to(dev)       # packed along N: 8 columns per word
        fused.qzeros = torch.cat([l.qzeros for l in linears], dim=1).to(dev)
        fused.scales = torch.cat([l.scales for l in linears], dim=1).to(dev)
        fused.bias = _cat_bias(linears)
        for l in linears:
            del l.qweight, l.qzeros, l.scales
    elif isinstance(first, SqW8A8BBF16OBF16PerChannel):
        dev = device if device is not None else first.qweight.device
        fused = SqW8A8BBF16OBF16PerChannel(first.w_bit, first.group_size, first.in_features, out_features, has_bias,
                                           dev=dev, dtype=first.dtype)
        fused.qweight = torch.cat([l.qweight for l in linears], dim=0).to(dev).contiguous()
        fused.weight_scale = torch.cat([l.weight_scale.reshape(-1) for l in linears], dim=0).to(dev).contiguous()
        fused.bias = _cat_bias(linears)
        for l in linears:
            del l.qweight, l.weight_scale
    else:                                                # FP8DynamicLinear, per token x per channel
        dev = device if device is not None else first.weight.device
        fused = FP8DynamicLinear(first.in_features, out_features, has_bias, dev=dev, dtype=first.dtype,
                                 qdtype=first.qdtype, per_tensor=False)
        P = torch.nn.Parameter
        fused.weight = P(torch.cat([l.weight.data for l in linears], dim=0).to(dev).contiguous(), requires_grad=False)
        fused.weight_scale = P(torch.cat([l.weight_scale.data.reshape(-1, 1) for l in linears], dim=0).to(dev).contiguous(),
                               requires_grad=False)
        b = _cat_bias(linears)
        fused.bias = P(b, requires_grad=False) if b is not None else None
        for l in linears:
            del l.weight, l.weight_scale
    return fused


def fuse_qkv(module, q_proj, k_proj, v_proj):
    """ref fused_utils.py:43-104: returns the fused qkv layer, or the tuple (q_proj, k_proj, v_proj)
    unchanged when the scheme cannot be fused."""
    if not (fusable(q_proj) and type(k_proj) is type(q_proj) and type(v_proj) is type(q_proj)):
        return (q_proj, k_proj, v_proj)
    try:
        dev = next(iter(module.state_dict().values())).device
    except (StopIteration, AttributeError):
        dev = None
    return fuse_linears([q_proj, k_proj, v_proj], dev)


class FusedGateUpMLP(torch.nn.Module):
    """down(silu(gate(x)) * up(x)) with gate and up fused into one projection and SiLU * up computed by
    one kernel (the data flow of HF's Qwen2MLP, which the reference keeps as separate torch ops)."""

    def __init__(self, gate_proj, up_proj, down_proj):
        super().__init__()
        self.gate_up = fuse_linears([gate_proj, up_proj]) if fusable(gate_proj) and type(up_proj) is type(gate_proj) else None
        self.gate_proj, self.up_proj = (None, None) if self.gate_up is not None else (gate_proj, up_proj)
        self.down_proj = down_proj

    @torch.no_grad()
    def forward(self, x):
        from . import glue
        if self.gate_up is not None:
            gu = self.gate_up(x)
        else:
            gu = torch.cat([self.gate_proj(x), self.up_proj(x)], dim=-1)
        h, _, _ = glue.silu_mul(gu)
        return self.down_proj(h)

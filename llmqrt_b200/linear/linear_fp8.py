"""FP8 e4m3 W8A8 linear layers (dynamic and static activation scales).

Names, constructor arguments, parameter names / shapes and `from_linear` follow
runtime/nn_models/modules/linear/linear_fp8.py.  The reference stores the pre-scaled weight as a
16-bit Parameter and casts all of it to fp8 on every forward (linear_fp8.py:188, :286); here the
fp8 copy is made once per weight version and kept.
"""
from __future__ import annotations

from typing import Tuple

import torch

from .. import ops
from .linear_base import LinearBase, tensor_key

dtype_to_str = {torch.bfloat16: "bfloat16", torch.float16: "float16"}


def per_tensor_quantize(tensor: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(e4m3 tensor, fp32 scale); ref linear_fp8.py:11-32."""
    q, scale = ops.quantize_fp8(tensor, per_token=False)
    return q.view(tensor.shape), scale.reshape(())


def static_per_tensor_quantize(tensor: torch.Tensor, scale) -> torch.Tensor:
    """e4m3(clamp(tensor / scale)); ref linear_fp8.py:34-37."""
    s = scale if isinstance(scale, torch.Tensor) else torch.tensor([scale], dtype=torch.float32, device=tensor.device)
    return ops.quantize_fp8_static(tensor, s).view(tensor.shape)


def per_token_quantize(tensor: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(e4m3 tensor, fp32 scales [..., 1]); ref linear_fp8.py:40-63."""
    if tensor.numel() == 0:
        return (torch.empty_like(tensor, dtype=torch.float8_e4m3fn),
                torch.ones((*tensor.shape[:-1], 1), dtype=torch.float32, device=tensor.device))
    q, scale = ops.quantize_fp8(tensor, per_token=True)
    return q.view(tensor.shape), scale.view(*tensor.shape[:-1], 1)


class _FP8Base(LinearBase):
    def _init_common(self, in_features, out_features, bias, dev, dtype, qdtype, per_channel_scale):
        self.dtype = dtype
        self.qdtype = qdtype
        self.in_features = in_features
        self.out_features = out_features
        P = torch.nn.Parameter
        self.weight = P(torch.randn((out_features, in_features), dtype=dtype, device=dev), requires_grad=False)
        shape = (out_features, 1) if per_channel_scale else (1,)
        self.weight_scale = P(torch.randn(shape, dtype=torch.float32, device=dev), requires_grad=False)
        self.bias = P(torch.zeros(out_features, dtype=dtype, device=dev), requires_grad=False) if bias else None
        self._qw_key = None
        self._qw = None

    def _fp8_weight(self) -> torch.Tensor:
        key = tensor_key(self.weight)
        if key != self._qw_key:
            self._qw = self.weight.data.to(self.qdtype).contiguous()       # [N, K] e4m3, made once
            self._qw_key = key
        return self._qw

    def _bias_for(self, dt):
        return None if self.bias is None else self.bias.data.to(dt)


class FP8DynamicLinear(_FP8Base):
    """Dynamic activation scale: per tensor (tensor-wise kernel) or per token (row-wise kernel).
    ref linear_fp8.py:134-223."""

    def __init__(self, in_features, out_features, bias, dev="cuda:0", dtype=torch.bfloat16,
                 qdtype=torch.float8_e4m3fn, per_tensor=True):
        super().__init__()
        self.per_tensor = per_tensor
        self._init_common(in_features, out_features, bias, dev, dtype, qdtype, per_channel_scale=not per_tensor)

    @classmethod
    def from_linear(cls, module: torch.nn.Linear, w_bit=8, group_size=0, init_only=True, dtype=torch.bfloat16,
                    per_tensor=True):
        assert group_size == 0, "not support group wise fp8 quant yet! pls set group_size = 0"
        layer = cls(in_features=module.in_features, out_features=module.out_features, bias=module.bias is not None,
                    dev=module.weight.device, dtype=dtype, per_tensor=per_tensor)
        if init_only:
            return layer
        w = module.weight.data.float()
        amax = w.abs().amax() if per_tensor else w.abs().amax(dim=1, keepdim=True)
        scale = amax.clamp(min=1e-12) / 448.0
        layer.weight.data.copy_((w / scale).clamp(-448, 448).to(dtype))
        layer.weight_scale.data.copy_(scale.reshape(layer.weight_scale.shape))
        if module.bias is not None:
            layer.bias.data.copy_(module.bias.data.to(dtype))
        return layer

    @torch.no_grad()
    def forward(self, x):
        assert x.device == self.weight.device, "when fp8 linear fwd, input and qweight must be same device!"
        x_shape = x.shape
        if x.shape[0] == 0 or x.numel() == 0:
            return torch.zeros(x.shape[:-1] + (self.out_features,), dtype=x.dtype, device=x.device)
        x2 = x.reshape(-1, x_shape[-1])
        qw = self._fp8_weight()
        if self.per_tensor:
            qx, x_scale = ops.quantize_fp8(x2, per_token=False)
            alpha = self.weight_scale.data.reshape(1) * x_scale                 # stays on the device
            out = ops.fp8_linear_tensorwise(qx, qw, self._bias_for(self.dtype), alpha, 1.0, self.dtype,
                                            static_weight=True)
        else:
            qx, x_scale = ops.quantize_fp8(x2, per_token=True)
            bias = self.bias.data if self.bias is not None else None
            if bias is not None and bias.dtype not in (torch.bfloat16, torch.float32):
                bias = bias.float()
            out = ops.fp8_linear_rowwise(qx, qw, bias, x_scale, self.weight_scale.data.reshape(1, -1),
                                         static_weight=True)
        return out.to(x.dtype).view(*x_shape[:-1], -1)


class FP8StaticLinear(_FP8Base):
    """Static per-tensor activation scale, optional fake-quantized output.  ref linear_fp8.py:226-313."""

    def __init__(self, in_features, out_features, bias, dev="cuda:0", dtype=torch.bfloat16,
                 qdtype=torch.float8_e4m3fn, per_tensor=True, quantize_output=False):
        super().__init__()
        self.per_tensor = per_tensor
        self._init_common(in_features, out_features, bias, dev, dtype, qdtype, per_channel_scale=False)
        P = torch.nn.Parameter
        self.input_scale = P(torch.randn(1, dtype=torch.float32, device=dev), requires_grad=False)
        self.quantize_output = quantize_output
        self.output_scale = P(torch.randn(1, dtype=torch.float32, device=dev), requires_grad=False)

    @classmethod
    def from_linear(cls, module: torch.nn.Linear, w_bit=8, group_size=0, init_only=True, dtype=torch.bfloat16,
                    per_tensor=True, quantize_output=False):
        assert group_size == 0, "not support group wise fp8 quant yet! pls set group_size = 0"
        layer = cls(in_features=module.in_features, out_features=module.out_features, bias=module.bias is not None,
                    dev=module.weight.device, dtype=dtype, per_tensor=True, quantize_output=quantize_output)
        if init_only:
            return layer
        w = module.weight.data.float()
        scale = w.abs().amax().clamp(min=1e-12) / 448.0
        layer.weight.data.copy_((w / scale).clamp(-448, 448).to(dtype))
        layer.weight_scale.data.fill_(float(scale))
        if module.bias is not None:
            layer.bias.data.copy_(module.bias.data.to(dtype))
        return layer

    @torch.no_grad()
    def forward(self, x):
        assert x.device == self.weight.device, "when fp8 linear fwd, input and qweight must be same device!"
        assert self.per_tensor, "[error!!] static activation quant only support per tensor!"
        x_shape = x.shape
        if x.shape[0] == 0 or x.numel() == 0:
            return torch.zeros(x.shape[:-1] + (self.out_features,), dtype=x.dtype, device=x.device)
        x2 = x.reshape(-1, x_shape[-1])
        qx = ops.quantize_fp8_static(x2, self.input_scale.data)
        alpha = self.weight_scale.data.reshape(1) * self.input_scale.data.reshape(1)
        out = ops.fp8_linear_tensorwise(qx, self._fp8_weight(), self._bias_for(self.dtype), alpha, 1.0, self.dtype,
                                        static_weight=True)
        out = out.view(*x_shape[:-1], -1)
        if self.quantize_output:
            qout = ops.quantize_fp8_static(out, self.output_scale.data).view(out.shape)
            out = qout.to(out.dtype) * self.output_scale.data
        return out.to(x.dtype)

"""SmoothQuant int8 W8A8 linear layers.

Class names, constructor arguments, buffer names / shapes and `from_linear` follow
runtime/nn_models/modules/linear/linear_sq.py so that state dicts load unchanged; `forward` keeps the
same arithmetic but runs it as two kernels (fused dynamic quantizer, GEMM with fused epilogue) with no
host synchronisation.
"""
from __future__ import annotations

import torch

from .. import ops
from .linear_base import LinearBase, tensor_key


def quantize_activation_per_tensor_absmax(t: torch.Tensor, n_bits: int = 8):
    """(int8 tensor, 0-d scale in t.dtype); ref linear_sq.py:44-53."""
    assert n_bits == 8
    q, scale, _ = ops.quantize_int8(t, per_token=False)
    return q.view(t.shape), scale


def quantize_activation_per_token_absmax(t: torch.Tensor, n_bits: int = 8):
    """(int8 tensor, [..., 1] scales in t.dtype); ref linear_sq.py:55-65."""
    assert n_bits == 8
    q, scale, _ = ops.quantize_int8(t, per_token=True)
    return q.view(t.shape), scale.view(*t.shape[:-1], 1)


class SqW8A8BBF16OBF16PerTensor(LinearBase):
    """Per-tensor weight scale, dynamic per-tensor activation scale (ref linear_sq.py:69-153).

    y = fp16(alpha * (xq @ wq^T) + bias), alpha = T(input_scale * weight_scale), returned in x's dtype
    (the kernel, like the reference's, computes an fp16 result).
    """

    def __init__(self, w_bit, group_size, in_features, out_features, bias, dev="cuda:0", dtype=torch.float16,
                 weight_scale=1.0, input_scale=1.0, alpha=1.0, beta=1.0):
        super().__init__()
        self.w_bit = w_bit
        self.group_size = group_size
        self.in_features = in_features
        self.out_features = out_features
        self.register_buffer("qweight", torch.randint(-127, 127, (out_features, in_features), dtype=torch.int8,
                                                      device=dev))
        if bias:
            self.register_buffer("bias", torch.zeros(out_features, dtype=dtype, device=dev))
        else:
            self.bias = None
        self.register_buffer("weight_scale", torch.tensor(weight_scale, device=dev))
        self.register_buffer("input_scale", torch.tensor(input_scale, device=dev))
        self._ws_key = None
        self._ws_value = 1.0
        self._bias_key = None
        self._bias_f16 = None

    def _weight_scale_value(self) -> float:
        # The reference calls weight_scale.item() on every forward; the value only changes when the
        # buffer is reloaded, so read it back once per buffer version.
        key = tensor_key(self.weight_scale)
        if key != self._ws_key:
            self._ws_value = float(self.weight_scale.item())
            self._ws_key = key
        return self._ws_value

    def _bias_as_f16(self, device) -> torch.Tensor:
        key = tensor_key(self.bias) if self.bias is not None else ("none", device)
        if key != self._bias_key:
            self._bias_f16 = (self.bias.to(torch.float16) if self.bias is not None
                              else torch.zeros(self.out_features, dtype=torch.float16, device=device))
            self._bias_key = key
        return self._bias_f16

    @torch.no_grad()
    def forward(self, x):
        assert x.device == self.qweight.device, "when sq linear fwd, input and qweight must be same device!"
        x_shape = x.shape
        x2 = x.reshape(-1, x_shape[-1])
        if x2.shape[0] == 0:
            return torch.zeros(*x_shape[:-1], self.out_features, dtype=x.dtype, device=x.device)
        qx, _, alpha = ops.quantize_int8(x2, per_token=False, scale_mul=self._weight_scale_value())
        y = ops.int8_linear_per_tensor(qx, self.qweight, self._bias_as_f16(x.device), alpha, 1.0, static_weight=True)
        return y.to(x.dtype).view(*x_shape[:-1], -1)

    @classmethod
    def from_linear(cls, module: torch.nn.Linear, w_bit, group_size, init_only=True, dtype=torch.float16,
                    per_tensor=True):
        layer = cls(w_bit=w_bit, group_size=group_size, in_features=module.in_features,
                    out_features=module.out_features, bias=module.bias is not None, dev=module.weight.device,
                    dtype=dtype)
        if init_only:
            return layer
        w = module.weight.data.float()
        scale = w.abs().max().clamp(min=1e-8) / 127
        layer.qweight.copy_(torch.round(w / scale).clamp(-128, 127).to(torch.int8))
        layer.weight_scale.copy_(scale)
        if module.bias is not None:
            layer.bias.copy_(module.bias.data.to(dtype))
        return layer


class SqW8A8BBF16OBF16PerChannel(LinearBase):
    """Per-output-channel weight scales, dynamic per-token activation scales, dequantization fused into
    the GEMM epilogue: y = T((acc * weight_scale[n]) * a_scale[m] + bias[n]).

    The reference sketches this class (linear_sq.py:155-214) around a kernel it never compiled
    (runtime/csrc/smoothquant/sq_gemm.h:19-24); buffers follow its intent: qweight [N, K] int8,
    weight_scale [N], bias [N].
    """

    def __init__(self, w_bit, group_size, in_features, out_features, bias, dev="cuda:0", dtype=torch.float16,
                 alpha=1.0, beta=1.0):
        super().__init__()
        self.w_bit = w_bit
        self.group_size = group_size
        self.in_features = in_features
        self.out_features = out_features
        self.dtype = dtype
        self.register_buffer("qweight", torch.randint(-127, 127, (out_features, in_features), dtype=torch.int8,
                                                      device=dev))
        if bias:
            self.register_buffer("bias", torch.zeros(out_features, dtype=dtype, device=dev))
        else:
            self.bias = None
        self.register_buffer("weight_scale", torch.ones(out_features, dtype=torch.float32, device=dev))

    @torch.no_grad()
    def forward(self, x):
        assert x.device == self.qweight.device, "when sq linear fwd, input and qweight must be same device!"
        x_shape = x.shape
        x2 = x.reshape(-1, x_shape[-1])
        if x2.shape[0] == 0:
            return torch.zeros(*x_shape[:-1], self.out_features, dtype=x.dtype, device=x.device)
        qx, _, a_scale = ops.quantize_int8(x2, per_token=True)
        y = ops.int8_linear_per_channel(qx, self.qweight, self.bias, a_scale, self.weight_scale, x.dtype,
                                        static_weight=True)
        return y.view(*x_shape[:-1], -1)

    def forward_quantized(self, qx: torch.Tensor, a_scale: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """GEMM + epilogue on activations a fused producer kernel has already quantized."""
        return ops.int8_linear_per_channel(qx, self.qweight, self.bias, a_scale, self.weight_scale, out_dtype,
                                           static_weight=True)

    @classmethod
    def from_linear(cls, module: torch.nn.Linear, w_bit, group_size, init_only=True, dtype=torch.float16,
                    per_tensor=False):
        layer = cls(w_bit=w_bit, group_size=group_size, in_features=module.in_features,
                    out_features=module.out_features, bias=module.bias is not None, dev=module.weight.device,
                    dtype=dtype)
        if init_only:
            return layer
        w = module.weight.data.float()
        scales = (w.abs().amax(dim=1).clamp(min=1e-8) / 127)
        layer.qweight.copy_(torch.round(w / scales[:, None]).clamp(-128, 127).to(torch.int8))
        layer.weight_scale.copy_(scales)
        if module.bias is not None:
            layer.bias.copy_(module.bias.data.to(dtype))
        return layer

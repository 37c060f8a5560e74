"""AWQ W4A16 linear layer.

Name, constructor arguments, buffer names / shapes / dtypes and `from_linear` follow
runtime/nn_models/modules/linear/linear_awq.py:78-267, so AWQ checkpoints load unchanged.  On the
first forward after the buffers change, the layer is repacked once into the K-major streaming layout
the CUDA kernels read; decode-sized inputs then stream the 4-bit weights directly, larger inputs
dequantize once and use the tcgen05 fp16 GEMM.
"""
from __future__ import annotations

import torch

from .. import ops
from .linear_base import LinearBase, tensor_key

AWQ_PACK_ORDER = [0, 2, 4, 6, 1, 3, 5, 7]


def _pack_awq(values: torch.Tensor) -> torch.Tensor:
    """uint4 values [R, N] -> int32 [R, N/8]; nibble i of a word holds column 8j + AWQ_PACK_ORDER[i]."""
    v = values.to(torch.int64).reshape(values.shape[0], -1, 8)
    word = torch.zeros(v.shape[:2], dtype=torch.int64, device=values.device)
    for i, src in enumerate(AWQ_PACK_ORDER):
        word |= (v[:, :, src] & 0xF) << (4 * i)
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word)
    return word.to(torch.int32)


class WQLinear_GEMM(LinearBase):
    def __init__(self, w_bit, group_size, in_features, out_features, bias, dev, training=False):
        super().__init__()
        if w_bit not in [4]:
            raise NotImplementedError("Only 4-bit are supported for now.")
        self.in_features = in_features
        self.out_features = out_features
        self.w_bit = w_bit
        self.group_size = group_size if group_size != -1 else in_features
        self.training = training
        assert self.in_features % self.group_size == 0
        assert out_features % (32 // self.w_bit) == 0
        pack = 32 // self.w_bit
        self.register_buffer("qweight", torch.zeros((in_features, out_features // pack), dtype=torch.int32, device=dev))
        self.register_buffer("qzeros", torch.zeros((in_features // self.group_size, out_features // pack),
                                                   dtype=torch.int32, device=dev))
        self.register_buffer("scales", torch.zeros((in_features // self.group_size, out_features),
                                                   dtype=torch.float16, device=dev))
        if bias:
            self.register_buffer("bias", torch.zeros(out_features, dtype=torch.float16, device=dev))
        else:
            self.bias = None
        self._packed_key = None
        self._packed = None

    @classmethod
    def from_linear(cls, linear, w_bit, group_size, init_only=False, dtype=torch.bfloat16, scales=None, zeros=None,
                    per_tensor=False):
        layer = cls(w_bit, group_size, linear.in_features, linear.out_features, linear.bias is not None,
                    linear.weight.device)
        if init_only:
            return layer
        # Real quantization (ref linear_awq.py:170-220): scales / zeros are [K/G, out_features];
        # q[k, n] = round((w[n, k] + zero * scale) / fp16(scale)), packed along N.
        assert scales is not None and zeros is not None
        G = layer.group_size
        dev = linear.weight.device
        scales, zeros = scales.to(dev), zeros.to(dev)
        layer.scales = scales.clone().half()
        scale_zeros = (zeros * scales).repeat_interleave(G, dim=0)                       # [K, N]
        s16 = layer.scales.repeat_interleave(G, dim=0)
        q = torch.round((linear.weight.data.t() + scale_zeros) / s16).to(torch.int32)    # [K, N]
        if linear.bias is not None:
            layer.bias = linear.bias.clone().half()
        layer.qweight = _pack_awq(q)
        layer.qzeros = _pack_awq(zeros.to(torch.int32))
        return layer

    def packed(self) -> ops.AwqPacked:
        key = tensor_key(self.qweight, self.qzeros, self.scales)
        if key != self._packed_key:
            self._packed = ops.AwqPacked(self.qweight, self.scales, self.qzeros)
            self._packed_key = key
        return self._packed

    @torch.no_grad()
    def forward(self, x):
        assert x.device == self.qweight.device, "when awq linear fwd, input and qweight must be same device!"
        out_shape = x.shape[:-1] + (self.out_features,)
        if x.shape[0] == 0 or x.numel() == 0:
            return torch.zeros(out_shape, dtype=x.dtype, device=x.device)
        input_dtype = x.dtype
        x16 = x if input_dtype == torch.float16 else x.to(torch.float16)
        out = ops.awq_gemm(x16.reshape(-1, self.in_features), self.packed(), self.bias)
        if input_dtype != torch.float16:
            out = out.to(input_dtype)
        return out.reshape(out_shape)

    def extra_repr(self) -> str:
        return "in_features={}, out_features={}, bias={}, w_bit={}, group_size={}".format(
            self.in_features, self.out_features, self.bias is not None, self.w_bit, self.group_size)

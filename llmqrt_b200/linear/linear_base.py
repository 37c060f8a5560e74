import torch


class LinearBase(torch.nn.Module):
    """Common base of the quantized linear layers (ref: runtime/nn_models/modules/linear/linear_base.py)."""

    def forward(self, x):
        raise NotImplementedError


def tensor_key(*tensors):
    """Identity + in-place-version key of tensors, used to invalidate caches derived from buffers."""
    return tuple((t.data_ptr(), t._version, tuple(t.shape), t.dtype, t.device) for t in tensors if t is not None)

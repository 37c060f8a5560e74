"""Contiguous KV cache with the reference's interface (runtime/nn_models/modules/nonlinear/cache.py:4-79)."""
import torch

from .. import attention


class WindowedCache:
    def __init__(self, cache_batch_size, n_heads, n_kv_heads, head_dim, max_seq_len, device):
        size = (cache_batch_size, max_seq_len, n_kv_heads if n_kv_heads != 0 else n_heads, head_dim)
        self.v = torch.zeros(size, device=device, dtype=torch.float16)
        self.k = torch.zeros(size, device=device, dtype=torch.float16)
        self.max_seq_len = max_seq_len

    def get_kv(self, batch_size, start_pos, seqlen):
        return self.v[:batch_size, : start_pos + seqlen], self.k[:batch_size, : start_pos + seqlen]

    def update_kv(self, values_store, keys_store, batch_size, start_pos, seqlen):
        """cache[:B, start:start+S] = store, as one kernel for both tensors."""
        attention.kv_append(self.k[:batch_size], self.v[:batch_size], keys_store.to(self.k.dtype),
                            values_store.to(self.v.dtype), cache_seqlens=None, start_pos=start_pos)

    def roll_kv_n_steps(self, start_pos, n=100):
        """Drops the n oldest positions.  The reference rolls dims=2 of the [B, S, H, D] tensors
        (cache.py:48-61), i.e. the head axis; this rolls the sequence axis, which is what the caller
        (prepare_cache, runtime/utils/fused_utils.py:12-25) means."""
        n = min(n, self.max_seq_len)
        self.v = torch.roll(self.v, shifts=-n, dims=1)
        self.k = torch.roll(self.k, shifts=-n, dims=1)
        self.v[:, -n:] = 0
        self.k[:, -n:] = 0
        return start_pos - n

    def to(self, device):
        """Accepts a device or, like the reference's call site (attn.py:274), a tensor to imitate."""
        if isinstance(device, torch.Tensor):
            self.k = self.k.to(device=device.device, dtype=device.dtype)
            self.v = self.v.to(device=device.device, dtype=device.dtype)
        else:
            self.k = self.k.to(device)
            self.v = self.v.to(device)

    def increase_batch_size(self, to_bsz):
        self.v = torch.zeros(to_bsz, *self.v.shape[1:], dtype=self.v.dtype, device=self.v.device)
        self.k = torch.zeros(to_bsz, *self.k.shape[1:], dtype=self.k.dtype, device=self.k.device)

    def decrease_batch_size(self, to_bsz):
        self.v = self.v[:to_bsz]
        self.k = self.k[:to_bsz]

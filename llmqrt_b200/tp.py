"""Host-side tensor-parallel logic: head placement, shard slicing, sampling reduction, and the handle
of the peer-buffer all-reduce (llmqrt_comm_* of the C ABI).

The reference has no tensor parallelism (its only multi-device mode is accelerate's layer placement,
runtime/core/base.py:213-221); this is the Megatron column/row scheme added around the quantized
linears: q/k/v/gate/up split by output channels, o_proj/down_proj by input channels with an allreduce
of the partial outputs.
"""
from __future__ import annotations

import torch


def head_assignment(num_heads: int, num_kv_heads: int, tp: int, rank: int) -> tuple[list[int], list[int]]:
    """Query heads and KV heads served by `rank`.

    tp dividing num_kv_heads: contiguous blocks of KV heads together with their whole query groups.
    tp a multiple of num_kv_heads: every KV head is replicated on tp/num_kv_heads ranks and its query
    group is split among them as evenly as possible (leading ranks get the extra head), e.g. 28 query /
    4 KV heads on 8 ranks -> 4 + 3 query heads per KV head.
    """
    if not (0 <= rank < tp):
        raise ValueError("rank out of range")
    rep = num_heads // num_kv_heads
    if num_kv_heads % tp == 0:
        per = num_kv_heads // tp
        kv = list(range(rank * per, (rank + 1) * per))
        return [h for j in kv for h in range(j * rep, (j + 1) * rep)], kv
    if tp % num_kv_heads != 0:
        raise ValueError(f"tensor parallel size {tp} must divide or be a multiple of {num_kv_heads} KV heads")
    share = tp // num_kv_heads
    if share > rep:
        raise ValueError("more ranks per KV head than query heads in its group")
    j, part = rank // share, rank % share
    base, extra = rep // share, rep % share
    start = part * base + min(part, extra)
    count = base + (1 if part < extra else 0)
    return [j * rep + start + i for i in range(count)], [j]


def rows_of_heads(heads: list[int], head_dim: int) -> list[int]:
    """Row (or column) indices of a projection matrix that belong to `heads`."""
    return [h * head_dim + i for h in heads for i in range(head_dim)]


def greedy_select(val: torch.Tensor, idx: torch.Tensor, tp: int, group=None) -> torch.Tensor:
    """Vocabulary-parallel greedy sampling: every rank holds the best (value, global token id) of its
    vocabulary shard per row; returns the global argmax per row (ties go to the lowest rank, i.e. the
    lowest token id, like a single argmax over the full vocabulary)."""
    if tp == 1:
        return idx
    vals = [torch.empty_like(val) for _ in range(tp)]
    idxs = [torch.empty_like(idx) for _ in range(tp)]
    torch.distributed.all_gather(vals, val.contiguous(), group=group)
    torch.distributed.all_gather(idxs, idx.contiguous(), group=group)
    vals, idxs = torch.stack(vals), torch.stack(idxs)
    best = vals.float().argmax(dim=0, keepdim=True)
    return idxs.gather(0, best)[0]


class PeerAllreduce:
    """Sum all-reduce of small 16-bit tensors over buffers that every rank of `group` maps from every
    other rank (one node, one process per GPU): llmqrt_comm_* of the C ABI.

    Construction is collective (an all-gather of the buffer handles and a barrier).  `allreduce` is
    in place, allocates nothing and can be captured in a CUDA graph; every rank must issue the same
    sequence of calls.  `check()` reads the sticky status the kernels raise when a bounded wait on a
    peer ran out (it synchronizes the device).
    """

    def __init__(self, device: torch.device, rank: int, world: int, max_bytes: int, group=None):
        import ctypes

        from . import _lib as L
        self._L, self.device, self.max_bytes, self.group = L, device, int(max_bytes), group
        self._comm = ctypes.c_void_p()
        with torch.cuda.device(device):
            L.call("llmqrt_comm_create", rank, world, self.max_bytes, ctypes.byref(self._comm))
            nbytes = L._lib.llmqrt_comm_handle_bytes()
            buf = ctypes.create_string_buffer(nbytes)
            L.call("llmqrt_comm_local_handle", self._comm, buf)
            mine = torch.tensor(list(buf.raw), dtype=torch.uint8, device=device)
            handles = [torch.empty_like(mine) for _ in range(world)]
            torch.distributed.all_gather(handles, mine, group=group)
            for peer in range(world):
                if peer != rank:
                    L.call("llmqrt_comm_open_peer", self._comm, peer, bytes(handles[peer].cpu().tolist()))
            torch.distributed.barrier(group=group)            # every buffer is mapped everywhere before first use

    @property
    def handle(self):
        """The opaque communicator pointer the llmqrt_comm_* entry points take."""
        return self._comm

    def eligible(self, x: torch.Tensor) -> bool:
        """Whether `x` goes over the peer buffers.  Depends on dtype and element count only -- facts
        every rank shares -- so all ranks take the same path (a rank that chose NCCL while the others
        polled the buffers would stall them until the wait limit)."""
        return x.dtype in (torch.float16, torch.bfloat16) and x.numel() % 8 == 0 and x.numel() * 2 <= self.max_bytes

    def fits_rows(self, M: int, H: int) -> bool:
        """Capacity rule of llmqrt_comm_allreduce_rmsnorm: a row occupies one tagged 16-byte word per
        four values, with the row's thread count rounded up to whole warps."""
        threads = (H // 8 + 31) // 32 * 32
        return H % 8 == 0 and H <= 8192 and M * threads * 32 <= 2 * ((self.max_bytes + 255) // 256 * 256)

    def allreduce(self, x: torch.Tensor) -> torch.Tensor:
        """In-place sum over the group.  A tensor that is not contiguous or not 16-byte aligned (a
        rank-local accident) is staged through an aligned copy rather than sent down another path."""
        L = self._L
        buf = x if (x.is_contiguous() and x.data_ptr() % 16 == 0) else x.contiguous().clone()
        with torch.cuda.device(self.device):
            L.call("llmqrt_comm_allreduce", self._comm, L.ptr(buf), L.ptr(buf), L.dtype_code(x.dtype), x.numel(),
                   L.stream(self.device))
        if buf is not x:
            x.copy_(buf)
        return x

    def close(self) -> None:
        """Unmaps the peers' buffers and frees this rank's.  Collective: every rank calls it, after its
        last all-reduce has completed (the barrier makes sure no peer still writes into the buffer)."""
        if self._comm is not None and self._comm.value:
            torch.cuda.synchronize(self.device)
            torch.distributed.barrier(group=self.group)
            self._L.call("llmqrt_comm_destroy", self._comm)
            self._comm = None

    def set_poll_limit_ms(self, ms: int) -> None:
        """Bound of the waits on peers for calls launched (or graphs captured) from now on."""
        self._L.call("llmqrt_comm_set_poll_limit_ms", self._comm, int(ms))

    def check(self) -> None:
        import ctypes
        status = ctypes.c_int32(0)
        with torch.cuda.device(self.device):
            self._L.call("llmqrt_comm_status", self._comm, ctypes.byref(status))
        if status.value != 0:
            raise RuntimeError("llmqrt_b200: a tensor-parallel peer did not deliver its partial sums in time")


def allreduce_sum(x: torch.Tensor, tp: int, group=None, comm: PeerAllreduce | None = None) -> torch.Tensor:
    """In-place sum of the row-parallel partial outputs over the tensor-parallel group: over the
    peer-mapped buffers of `comm` when the tensor fits them, else NCCL (the choice depends only on the
    tensor's size, so all ranks take the same path)."""
    if tp > 1:
        if comm is not None and comm.eligible(x):
            comm.allreduce(x)
        else:
            torch.distributed.all_reduce(x, group=group)
    return x

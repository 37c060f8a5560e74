"""Host-side tensor-parallel logic (no kernels): head placement, shard slicing, sampling reduction.

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


def allreduce_sum(x: torch.Tensor, tp: int, group=None) -> torch.Tensor:
    """In-place sum of the row-parallel partial outputs over the tensor-parallel group."""
    if tp > 1:
        torch.distributed.all_reduce(x, group=group)
    return x

"""Host-side tensor-parallel logic: head placement, shard slicing, sampling reduction, and the handle
of the peer-buffer all-reduce (llmqrt_comm_* of the C ABI).

The reference has no tensor parallelism (its only multi-device mode is accelerate's layer placement,
runtime/core/base.py:213-221); this is the Megatron column/row scheme added around the quantized
linears: q/k/v/gate/up split by output channels, o_proj/down_proj by input channels with an allreduce
of the partial outputs.
"""
from __future__ import annotations

import os

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


# ---------------------------------------------------------------------------------------------
# Sharding of a loaded state dict (buffer names and layouts of the reference's linear classes:
# runtime/nn_models/modules/linear/linear_awq.py:97-131, linear_sq.py:77-88, linear_fp8.py:152-164;
# the loader that fills them: runtime/core/base.py:306-340)
# ---------------------------------------------------------------------------------------------
def split_points(total: int, parts: int, unit: int = 1) -> list[int]:
    """Boundaries 0 = b[0] <= ... <= b[parts] = total, every one a multiple of `unit`, as even as the
    unit allows (the leading parts get the extra units).  E.g. the 18944 input channels of Qwen2-7B's
    down_proj in AWQ groups of 128 on 8 ranks: 148 groups -> 19,19,19,19,18,18,18,18 groups."""
    if total % unit:
        raise ValueError(f"{total} is not a multiple of the unit {unit}")
    units = total // unit
    base, extra = divmod(units, parts)
    out = [0]
    for i in range(parts):
        out.append(out[-1] + (base + (1 if i < extra else 0)) * unit)
    return out


def _as_index(sel, size: int) -> torch.Tensor:
    if isinstance(sel, tuple):
        return torch.arange(sel[0], sel[1])
    idx = torch.as_tensor(sel, dtype=torch.int64).reshape(-1)
    if idx.numel() and (int(idx.min()) < 0 or int(idx.max()) >= size):
        raise ValueError("shard selection out of range")
    return idx


def _whole_blocks(idx: torch.Tensor, block: int, what: str) -> torch.Tensor:
    """`idx` must consist of whole aligned runs of `block` consecutive values; returns the run numbers."""
    if idx.numel() % block:
        raise ValueError(f"{what}: selection must cover whole blocks of {block}")
    runs = idx.reshape(-1, block)
    if not (torch.equal(runs[:, 0] % block, torch.zeros_like(runs[:, 0])) and
            torch.equal(runs, runs[:, :1] + torch.arange(block))):
        raise ValueError(f"{what}: selection must cover whole aligned blocks of {block}")
    return runs[:, 0] // block


def shard_linear_state(state: dict, method: str, mode: str, sel, keep_bias: bool = True) -> dict:
    """The shard of one quantized linear layer's state dict for Megatron tensor parallelism.

    method: "awq" | "sq" | "fp8_static_quant" | "fp8_dynamic_quant" (the registry keys of
            linear.method_to_linear).
    mode:   "column" -- `sel` selects OUTPUT channels (q/k/v by heads, gate, up): weight rows, per-channel
            scales and bias follow;  "row" -- `sel` selects INPUT channels (o_proj, down_proj): the
            partial outputs of the ranks are summed afterwards, per-channel scales are replicated and
            the bias is kept on one rank only (keep_bias).
    sel:    (start, stop) or a 1-D index list / tensor (e.g. tp.rows_of_heads(...) for head-wise splits).
    AWQ constraints: output channels travel in packed words of 8 columns, input channels in
    quantization groups, so selections must cover whole aligned blocks of 8 (column) or of the group
    size (row); split_points(..., unit=group_size) yields such row boundaries.
    Per-tensor scalars (SmoothQuant per-tensor weight / input scales, FP8 per-tensor scales) are copied.
    """
    out = {}
    if mode not in ("column", "row"):
        raise ValueError("mode must be 'column' or 'row'")
    if method == "awq":
        qweight, qzeros, scales = state["qweight"], state["qzeros"], state["scales"]
        K, N = qweight.shape[0], scales.shape[1]
        G = K // scales.shape[0]
        if mode == "column":
            idx = _as_index(sel, N)
            words = _whole_blocks(idx, 8, "awq column shard")
            out["qweight"], out["qzeros"], out["scales"] = qweight[:, words], qzeros[:, words], scales[:, idx]
        else:
            idx = _as_index(sel, K)
            groups = _whole_blocks(idx, G, "awq row shard")
            out["qweight"], out["qzeros"], out["scales"] = qweight[idx], qzeros[groups], scales[groups]
        n_axis = idx if mode == "column" else None
    elif method in ("sq", "fp8_static_quant", "fp8_dynamic_quant"):
        wname = "qweight" if method == "sq" else "weight"
        w = state[wname]
        N, K = w.shape
        idx = _as_index(sel, N if mode == "column" else K)
        out[wname] = w[idx] if mode == "column" else w[:, idx]
        ws = state["weight_scale"]
        out["weight_scale"] = (ws.reshape(N, -1)[idx].reshape((-1,) + tuple(ws.shape[1:]))
                               if (mode == "column" and ws.numel() == N and N > 1) else ws)
        for name in ("input_scale", "output_scale"):
            if name in state:
                out[name] = state[name]
        n_axis = idx if mode == "column" else None
    else:
        raise ValueError(f"unknown quantization method {method!r}")
    bias = state.get("bias")
    if bias is not None:
        if n_axis is not None:
            out["bias"] = bias[n_axis]
        else:
            out["bias"] = bias if keep_bias else torch.zeros_like(bias)
    return {k: (v.contiguous() if isinstance(v, torch.Tensor) else v) for k, v in out.items()}


def shard_decoder_layer(layer_state: dict, method: str, num_heads: int, num_kv_heads: int, head_dim: int, tp: int,
                        rank: int, prefix_map: dict | None = None) -> dict:
    """Shards the seven linears of one Qwen2-style decoder layer: q/k/v by heads (head_assignment), gate/up by
    output channels, o_proj / down_proj by the matching input channels.  `layer_state` maps the
    projection names ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj") to
    the state dicts of the layers; returns the same structure for this rank.  The intermediate
    dimension is cut on multiples of the AWQ group size (or 16 for the 8-bit schemes)."""
    names = prefix_map or {k: k for k in ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")}
    q_heads, kv_heads = head_assignment(num_heads, num_kv_heads, tp, rank)
    q_idx, kv_idx = rows_of_heads(q_heads, head_dim), rows_of_heads(kv_heads, head_dim)
    down = layer_state[names["down_proj"]]
    if method == "awq":
        inter = down["qweight"].shape[0]
        unit = inter // down["scales"].shape[0]
    else:
        inter = down["qweight" if method == "sq" else "weight"].shape[1]
        unit = 16
    b = split_points(inter, tp, unit)
    mlp = (b[rank], b[rank + 1])
    out = {
        names["q_proj"]: shard_linear_state(layer_state[names["q_proj"]], method, "column", q_idx),
        names["k_proj"]: shard_linear_state(layer_state[names["k_proj"]], method, "column", kv_idx),
        names["v_proj"]: shard_linear_state(layer_state[names["v_proj"]], method, "column", kv_idx),
        names["o_proj"]: shard_linear_state(layer_state[names["o_proj"]], method, "row", q_idx, keep_bias=rank == 0),
        names["gate_proj"]: shard_linear_state(layer_state[names["gate_proj"]], method, "column", mlp),
        names["up_proj"]: shard_linear_state(layer_state[names["up_proj"]], method, "column", mlp),
        names["down_proj"]: shard_linear_state(down, method, "row", mlp, keep_bias=rank == 0),
    }
    return out


def greedy_select(val: torch.Tensor, idx: torch.Tensor, tp: int, group=None) -> torch.Tensor:
    """Vocabulary-parallel greedy sampling: every rank holds the best (value, global token id) of its
    vocabulary shard per row; returns the global argmax per row (ties go to the lowest rank, i.e. the
    lowest token id, like a single argmax over the full vocabulary)."""
    if tp == 1:
        return idx
    # one collective: (value, token id) pairs as fp32 (token ids below 2^24 are exact in fp32)
    if int(idx.numel()) and val.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise TypeError("greedy_select: values must be floating point")
    mine = torch.stack([val.float(), idx.float()], dim=-1).contiguous()            # [B, 2]
    parts = [torch.empty_like(mine) for _ in range(tp)]
    torch.distributed.all_gather(parts, mine, group=group)
    both = torch.stack(parts)                                                      # [tp, B, 2]
    best = both[..., 0].argmax(dim=0, keepdim=True)                                # first maximum = lowest rank
    return both[..., 1].gather(0, best)[0].to(idx.dtype)


class PushedPartial:
    """Stands for partial sums that a GEMM has already sent to the peers (`PeerAllreduce.linear_push`)."""

    def __init__(self, M: int, H: int, dtype):
        self.M, self.H, self.dtype = M, H, dtype


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

    def push_ok(self, M: int, H: int) -> bool:
        """Whether a row-parallel int8 linear with M tokens and H outputs can send its results from the
        GEMM's epilogue (`linear_push`): shapes only, so that every rank decides alike."""
        if os.environ.get("LLMQRT_TP_PUSH", "1") == "0":           # A/B switch: the GEMM writes a tensor, the RMSNorm pushes
            return False
        return 16 < M <= 128 and self.fits_rows(M, H)

    def linear_push(self, a, w, bias, a_scale, w_scale, out_dtype, static_weight: bool = False) -> "PushedPartial":
        """int8 per-token x per-channel linear of a row-parallel layer whose 16-bit results go, from the
        GEMM's epilogue, straight into the peers' all-reduce buffers.  The returned token must be handed
        to `glue.rmsnorm(..., residual=token, comm=self)`, which gathers and sums (every rank alike)."""
        L = self._L
        M, K = a.shape
        N = w.shape[0]
        if not self.push_ok(M, N):
            raise RuntimeError("linear_push: shape outside the pushing schedule (16 < M <= 128, M x N within capacity)")
        a_s = a_scale.to(torch.float32).reshape(-1).contiguous()
        w_s = w_scale.to(torch.float32).reshape(-1).contiguous()
        if a_s.numel() != M or w_s.numel() != N:
            raise RuntimeError("linear_push: a_scale must have M elements and w_scale N elements")
        with torch.cuda.device(self.device):
            L.call("llmqrt_comm_int8_linear_per_channel", self._comm, L.ptr(a), a.stride(0), L.ptr(w), w.stride(0),
                   L.ptr(bias), L.dtype_code(bias.dtype) if bias is not None else L.F16, L.ptr(a_s), L.ptr(w_s),
                   L.dtype_code(out_dtype), M, N, K, L.ptr(L.workspace(self.device)), L.stream(self.device),
                   L.GEMM_STATIC_WEIGHT if static_weight else 0)
        return PushedPartial(M, N, out_dtype)

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

"""ctypes binding of libllmqrt_b200.so (the C ABI declared in include/llmqrt_b200.h).

The library is the only compute path of this package: if it cannot be loaded the import fails
loudly; there is no eager / CPU fallback.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libllmqrt_b200.so")

F16, BF16, F32, E4M3, E5M2 = 0, 1, 2, 3, 4
_DTYPE_CODE = {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32,
               torch.float8_e4m3fn: E4M3, torch.float8_e5m2: E5M2}


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        from . import build as _build
        _build.build()
    return ctypes.CDLL(LIB_PATH)


_lib = _load()

P, I64, I32, F, SZ = c_void_p, c_int64, c_int, c_float, c_size_t
_PROTOS = {
    "llmqrt_last_error": (c_char_p, []),
    "llmqrt_abi_version": (c_int, []),
    "llmqrt_launch_count": (ctypes.c_longlong, []),
    "llmqrt_workspace_bytes": (SZ, []),
    "llmqrt_set_gemm_path": (c_int, [I32]),
    "llmqrt_quantize_int8": (c_int, [P, I32, I64, I64, I64, I32, P, P, P, F, P, P]),
    "llmqrt_quantize_fp8": (c_int, [P, I32, I64, I64, I64, I32, P, P, F, P, P]),
    "llmqrt_quantize_fp8_static": (c_int, [P, I32, I64, I64, I64, P, P, P]),
    "llmqrt_w8a8_int8_linear_per_tensor": (c_int, [P, I64, P, I64, P, F, P, F, P, I64, I64, I64, I64, P, P, I32]),
    "llmqrt_w8a8_int8_linear_per_channel": (c_int, [P, I64, P, I64, P, I32, P, P, P, I32, I64, I64, I64, I64, P, P, I32]),
    "llmqrt_w8a8_int8_linear_per_channel_noalloc": (c_int, [P, I64, P, I64, P, I32, P, P, P, I32, I64, I64, I64, I64, P]),
    "llmqrt_w8a8_int8_gemm_s32": (c_int, [P, I64, P, I64, P, I64, I64, I64, I64, P, P, I32]),
    "llmqrt_f8f8_tensorwise": (c_int, [P, I32, I64, P, I64, P, F, P, F, P, I32, I64, I64, I64, I64, P, P, I32]),
    "llmqrt_f8f8bf16_rowwise": (c_int, [P, I32, I64, P, I64, P, I32, P, P, P, I64, I64, I64, I64, P, P, I32]),
    "llmqrt_awq_dequantize": (c_int, [P, P, P, I64, I64, I64, P, P]),
    "llmqrt_awq_repack": (c_int, [P, P, P, I64, I64, I64, P, P, P]),
    "llmqrt_awq_gemm": (c_int, [P, I64, P, P, P, P, I64, I64, I64, I64, I64, P, P]),
    "llmqrt_awq_dequantize_t": (c_int, [P, P, I64, I64, I64, P, P]),
    "llmqrt_gemm_16bit": (c_int, [P, I64, P, I64, P, P, I64, I32, I64, I64, I64, P, P]),
    "llmqrt_kv_append": (c_int, [P, P, I64, I64, P, P, P, c_int32, I32, I64, I64, I64, I64, I64, P]),
    "llmqrt_attn_decode": (c_int, [P, I64, P, P, I64, I64, P, P, P, P, I32, I64, I64, I64, I64, I64, F, P, P]),
    "llmqrt_attn_decode_append": (c_int, [P, I64, P, P, I64, P, P, I64, P, P, I64, I64, P, P, P, P, I32, I64, I64,
                                          I64, I64, I64, F, P, P]),
    "llmqrt_attn_prefill":(c_int, [P, I64, P, P, I64, P, I64, I32, I64, I64, I64, I64, I64, I32, F, P]),
    "llmqrt_rmsnorm": (c_int, [P, P, P, P, F, P, P, P, I32, I64, I64, P]),
    "llmqrt_rope_kv_write": (c_int, [P, I64, P, P, I64, P, P, I64, I64, c_int32, P, P, P, I64, I32, I64, I64, I64,
                                     I64, I64, P]),
    "llmqrt_silu_mul": (c_int, [P, I64, P, P, P, I32, I64, I64, P]),
    "llmqrt_comm_create": (c_int, [I32, I32, I64, ctypes.POINTER(c_void_p)]),
    "llmqrt_comm_handle_bytes": (c_int, []),
    "llmqrt_comm_local_handle": (c_int, [P, P]),
    "llmqrt_comm_open_peer": (c_int, [P, I32, P]),
    "llmqrt_comm_allreduce": (c_int, [P, P, P, I32, I64, P]),
    "llmqrt_comm_allreduce_rmsnorm": (c_int, [P, P, P, P, P, F, P, P, P, I32, I64, I64, P]),
    "llmqrt_comm_int8_linear_per_channel": (c_int, [P, P, I64, P, I64, P, I32, P, P, I32, I64, I64, I64, P, P, I32]),
    "llmqrt_comm_set_poll_limit_ms": (c_int, [P, c_int32]),
    "llmqrt_comm_status": (c_int, [P, ctypes.POINTER(ctypes.c_int32)]),
    "llmqrt_comm_destroy": (c_int, [P]),
}

EXPORTS = tuple(_PROTOS)


def _bind(lib: ctypes.CDLL) -> list[str]:
    missing = []
    for name, (res, args) in _PROTOS.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            missing.append(name)
            continue
        fn.restype = res
        fn.argtypes = args
    return missing


ABI_VERSION = 5          # llmqrt_abi_version() of the sources these prototypes describe

_missing = _bind(_lib)
if not _missing and _lib.llmqrt_abi_version() != ABI_VERSION:
    _missing = ["llmqrt_abi_version == %d" % ABI_VERSION]
if _missing:
    # A library built from older sources: rebuild once (needs nvcc) and load the fresh file.
    import _ctypes
    from . import build as _build
    _ctypes.dlclose(_lib._handle)
    _build.build()
    _lib = ctypes.CDLL(LIB_PATH)
    _missing = _bind(_lib)
    if not _missing and _lib.llmqrt_abi_version() != ABI_VERSION:
        _missing = ["llmqrt_abi_version == %d" % ABI_VERSION]
    if _missing:
        raise ImportError(f"{LIB_PATH} lacks symbols {_missing}; rebuild with `python llmqrt_b200/build.py --force`")


def last_error() -> str:
    return _lib.llmqrt_last_error().decode()


def check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(f"llmqrt_b200: {last_error()} (status {rc})")


def call(name: str, *args) -> None:
    check(getattr(_lib, name)(*args))


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise TypeError(f"llmqrt_b200: unsupported dtype {dt}") from None


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def stream(device: torch.device):
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("llmqrt_b200: tensors must live on a CUDA device (there is no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError("llmqrt_b200: all tensors must be on the same device")
    return dev


WORKSPACE_BYTES = int(_lib.llmqrt_workspace_bytes())
_ws_lock = threading.Lock()
_workspaces: dict[int, torch.Tensor] = {}


def workspace(device: torch.device) -> torch.Tensor:
    """Scratch buffer of `device`: zero-filled once, then owned by the kernels.

    One buffer per device: calls of this package on the same device must be ordered (one stream, or
    streams that depend on each other), because kernels that split their reduction share it.
    """
    key = device.index if device.index is not None else torch.cuda.current_device()
    ws = _workspaces.get(key)
    if ws is None:
        with _ws_lock:
            ws = _workspaces.get(key)
            if ws is None:
                ws = torch.zeros(WORKSPACE_BYTES, dtype=torch.uint8, device=device)
                _workspaces[key] = ws
    return ws


# Byte offset, inside a workspace, of the word a kernel sets to 1 when one of its bounded waits ran out.
STATUS_OFFSET = 64 * 1024 - 64 * 4 + 4


def kernel_status(device: torch.device) -> int:
    """Reads (synchronously) the bounded-wait status word of the current stream's workspace."""
    ws = workspace(device)
    return int(ws[STATUS_OFFSET:STATUS_OFFSET + 4].view(torch.int32).item())


def launch_count() -> int:
    """Kernels launched by the library so far in this process."""
    return int(_lib.llmqrt_launch_count())


GEMM_STATIC_WEIGHT = 1   # LLMQRT_GEMM_STATIC_WEIGHT of the header


def set_gemm_path(path: int) -> None:
    """0 = automatic, 1 = register-operand streaming kernel, 2 = tcgen05 kernel (tests / benchmarks)."""
    call("llmqrt_set_gemm_path", path)

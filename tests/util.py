"""Helpers shared by the tests: fixture loading and error metrics."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

_DT = {"torch.float16": torch.float16, "torch.bfloat16": torch.bfloat16,
       "torch.float8_e4m3fn": torch.float8_e4m3fn, "torch.float8_e5m2": torch.float8_e5m2}


def load_golden(name: str) -> dict:
    """Load tests/golden/<name>.npz, rebuilding 16-bit / fp8 tensors from their bit patterns."""
    raw = np.load(os.path.join(GOLDEN, name + ".npz"))
    out = {}
    for k in raw.files:
        if k.endswith("_dtype"):
            continue
        if k.endswith("_bits"):
            base = k[:-5]
            dt = _DT[str(raw[base + "_dtype"])]
            arr = raw[k]
            if arr.dtype == np.uint16:
                out[base] = torch.from_numpy(arr.view(np.int16).copy()).view(dt)
            else:
                out[base] = torch.from_numpy(arr.copy()).view(dt)
        else:
            a = raw[k]
            out[k] = torch.from_numpy(a.copy()) if a.ndim else a.item()
    return out


def rel_fro(a: torch.Tensor, b: torch.Tensor) -> float:
    """Relative Frobenius error ||a-b|| / ||b|| in fp64."""
    a = a.detach().cpu().to(torch.float64)
    b = b.detach().cpu().to(torch.float64)
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def max_abs(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.detach().cpu().to(torch.float64) - b.detach().cpu().to(torch.float64)).abs().max())


def bits_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    a = a.detach().cpu().contiguous()
    b = b.detach().cpu().contiguous()
    if a.dtype != b.dtype or a.shape != b.shape:
        return False
    if a.element_size() == 2:
        return bool((a.view(torch.int16) == b.view(torch.int16)).all())
    if a.element_size() == 1:
        return bool((a.view(torch.uint8) == b.view(torch.uint8)).all())
    return bool((a == b).all())


def ulp_mismatch_fraction(a: torch.Tensor, b: torch.Tensor):
    """(fraction of elements whose 16-bit patterns differ, max pattern distance)."""
    ai = a.detach().cpu().contiguous().view(torch.int16).to(torch.int32)
    bi = b.detach().cpu().contiguous().view(torch.int16).to(torch.int32)
    d = (ai - bi).abs()
    return float((d != 0).float().mean()), int(d.max())

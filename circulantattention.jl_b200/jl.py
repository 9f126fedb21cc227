"""Julia-shaped tensors.

The reference's arrays are column-major `(H, W, C, B)` CuArrays.  On the Python
side the same bytes are a torch tensor whose `.shape` is the Julia shape and
whose strides are column-major, so code and tests read like the reference's
(`q = jl.randn(128, 96, 64, 2)`), and `tensor.data_ptr()` can be handed to the
C ABI unchanged.
"""
from __future__ import annotations

import numpy as np
import torch


def _rev(n):
    return tuple(range(n - 1, -1, -1))


def is_colmajor(t: torch.Tensor) -> bool:
    """True when the strides are those of a dense column-major array (extent-1 dims may carry any stride)."""
    expect = 1
    for n, st in zip(t.shape, t.stride()):
        if n != 1 and st != expect:
            return False
        expect *= n
    return True


def colmajor(t: torch.Tensor) -> torch.Tensor:
    """`t` itself if it already is column-major, else a column-major copy."""
    if is_colmajor(t):
        return t
    r = _rev(t.ndim)
    return t.permute(r).contiguous().permute(r)


def empty(shape, dtype=torch.float32, device="cuda") -> torch.Tensor:
    shape = tuple(int(s) for s in shape)
    return torch.empty(tuple(reversed(shape)), dtype=dtype, device=device).permute(_rev(len(shape)))


def zeros(shape, dtype=torch.float32, device="cuda") -> torch.Tensor:
    shape = tuple(int(s) for s in shape)
    return torch.zeros(tuple(reversed(shape)), dtype=dtype, device=device).permute(_rev(len(shape)))


def ones(shape, dtype=torch.float32, device="cuda") -> torch.Tensor:
    shape = tuple(int(s) for s in shape)
    return torch.ones(tuple(reversed(shape)), dtype=dtype, device=device).permute(_rev(len(shape)))


def randn(*shape, dtype=torch.float32, device="cuda", generator=None) -> torch.Tensor:
    """Like `CUDA.randn(T, dims...)`; complex draws have unit variance (re, im ~ N(0, 1/2))."""
    t = torch.randn(tuple(reversed(shape)), dtype=dtype, device=device, generator=generator)
    return t.permute(_rev(len(shape)))


def from_numpy(a: np.ndarray, device="cuda", dtype=None) -> torch.Tensor:
    """numpy array with Julia logical shape -> column-major torch tensor."""
    a = np.asarray(a)
    t = torch.from_numpy(np.ascontiguousarray(a.T))
    if dtype is not None:
        t = t.to(dtype)
    return t.to(device).permute(_rev(a.ndim))


def to_numpy(t: torch.Tensor) -> np.ndarray:
    """Column-major torch tensor -> numpy array with the same (Julia) shape."""
    t = colmajor(t.detach())
    return t.permute(_rev(t.ndim)).contiguous().cpu().numpy().T


def reshape(t: torch.Tensor, *shape) -> torch.Tensor:
    """Julia `reshape` (column-major): a view when `t` is column-major."""
    shape = list(shape[0]) if len(shape) == 1 and isinstance(shape[0], (tuple, list)) else list(shape)
    n = t.numel()
    if shape.count(-1) == 1:
        known = int(np.prod([s for s in shape if s != -1])) if len(shape) > 1 else 1
        shape[shape.index(-1)] = n // max(known, 1)
    t = colmajor(t)
    if not (torch.is_grad_enabled() and t.requires_grad):
        # nothing to differentiate through: one strided view of the same column-major memory
        strides, acc = [], 1
        for n_ in shape:
            strides.append(acc)
            acc *= n_
        return t.as_strided(tuple(shape), tuple(strides), t.storage_offset())
    flat = t.permute(_rev(t.ndim)).reshape(tuple(reversed(shape)))
    return flat.permute(_rev(len(shape)))

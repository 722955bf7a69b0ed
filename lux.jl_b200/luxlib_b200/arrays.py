"""Julia-style (column-major) device arrays on top of torch tensors.

A "Julia array" here is a torch tensor whose logical shape is the Julia shape and whose strides are
column-major (first index contiguous), i.e. exactly the memory a CuArray of that shape has. torch
is only the allocator / stream provider."""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from . import _cabi


def colmajor_strides(shape: Sequence[int]):
    st, acc = [], 1
    for d in shape:
        st.append(acc)
        acc *= max(int(d), 1)
    return tuple(st)


def jl_empty(shape: Sequence[int], dtype: torch.dtype, device) -> torch.Tensor:
    """similar(x, T, shape...): uninitialised column-major array."""
    shape = tuple(int(d) for d in shape)
    return torch.empty_strided(shape, colmajor_strides(shape), dtype=dtype, device=device)


def jl_zeros(shape, dtype, device) -> torch.Tensor:
    t = jl_empty(shape, dtype, device)
    t.zero_()
    return t


def is_colmajor(t: torch.Tensor) -> bool:
    if t.numel() == 0:
        return True
    exp = colmajor_strides(t.shape)
    return all(s == e or d == 1 for s, e, d in zip(t.stride(), exp, t.shape))


def as_colmajor(t: torch.Tensor) -> torch.Tensor:
    """Returns `t` itself when already column-major, else a column-major copy (what the Julia side
    does for views before handing a pointer over)."""
    if is_colmajor(t):
        return t
    out = jl_empty(t.shape, t.dtype, t.device)
    out.copy_(t)
    return out


def jl_reshape(t: torch.Tensor, shape: Sequence[int]) -> torch.Tensor:
    """Julia's reshape: the same column-major memory under a new shape (torch's own reshape walks indices in row-major
    order and would permute the elements of a column-major tensor)."""
    t = as_colmajor(t)
    return torch.as_strided(t, tuple(shape), colmajor_strides(tuple(shape)), t.storage_offset())


def from_numpy(a: np.ndarray, device="cuda", dtype: torch.dtype | None = None) -> torch.Tensor:
    """Host numpy array (any layout, Julia index order) -> column-major device array."""
    a = np.asarray(a)
    rev = tuple(reversed(range(a.ndim)))
    t = torch.from_numpy(np.ascontiguousarray(a.transpose(rev)))  # C-order of reversed axes == column-major
    if dtype is not None:
        t = t.to(dtype)
    t = t.to(device)
    return t.permute(rev) if a.ndim > 1 else t


def to_numpy(t: torch.Tensor) -> np.ndarray:
    """Device array -> host numpy array (float32 for bf16), Julia index order."""
    t = t.detach()
    if t.dtype == torch.bfloat16:
        t = t.to(torch.float32)
    return t.cpu().numpy()


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return _cabi.F32
    if dt == torch.bfloat16:
        return _cabi.BF16
    raise _cabi.LuxLibB200Error(_cabi.UNSUPPORTED_DTYPE, f"{dt} is not handled by the B200 path (Float32 and BFloat16 only)")


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def current_stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def workspace(nbytes: int, device) -> torch.Tensor | None:
    """Caller-side scratch (the Julia shim uses `similar(x, UInt8, n)`); 256-byte aligned by the
    torch allocator."""
    if nbytes <= 0:
        return None
    return torch.empty(int(nbytes), dtype=torch.uint8, device=device)

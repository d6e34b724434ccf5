"""``triton_max`` / ``triton_min``: max / min along one axis, with indices.

Drop-ins for ``mdy_triton/core/triton_maxmin.py:66-97`` and ``:149-179`` (exported by
``core/__init__.py:6``; no patch module uses them).  Same call: ``(tensor, axis=-1, keepdim=False)`` and
a result object with ``values``, ``indices`` (int64) and ``func_type``.  One CUDA kernel
(``csrc/maxmin.cu``) instead of the reference's short-row / long-row Triton pair.  Where the reference
leaves it open, the result follows ``torch.max`` / ``torch.min``: the index is the first position of the
extreme, a NaN wins, and ``keepdim`` keeps the axis on the indices too (the reference un-squeezes only
the values).  No gradient is defined, as in the reference.
"""
from __future__ import annotations

import torch

from .. import _C


class VALUES_INDICES:
    """Result of :func:`triton_max` / :func:`triton_min` (reference ``triton_maxmin.py:5-15``); also
    unpacks like the ``(values, indices)`` pair torch returns."""

    def __init__(self, values, indices, func_type):
        self.values = values
        self.indices = indices
        self.func_type = func_type

    def __iter__(self):
        return iter((self.values, self.indices))

    def __repr__(self):
        return f"func_type={self.func_type}\nvalues={self.values}\nindices={self.indices})"

    __str__ = __repr__


def _extreme(tensor: torch.Tensor, axis: int, keepdim: bool, take_min: bool) -> VALUES_INDICES:
    _C.require_cuda(tensor)
    if tensor.dim() == 0:
        raise ValueError("triton_max / triton_min need at least one dimension")
    moved = torch.movedim(tensor.detach(), axis, -1)
    lead, n = moved.shape[:-1], moved.shape[-1]
    if n == 0:
        raise ValueError("cannot reduce over an empty axis")
    rows = moved.reshape(-1, n)
    if rows.stride(1) != 1 or (rows.shape[0] > 1 and rows.stride(0) < n):
        rows = rows.contiguous()
    m = rows.shape[0]
    values = torch.empty(m, dtype=tensor.dtype, device=tensor.device)
    indices = torch.empty(m, dtype=torch.int64, device=tensor.device)
    if m:
        with torch.cuda.device(tensor.device):
            _C.check(_C.lib().mdy_rowwise_extreme(_C.ptr(rows), _C.ptr(values), _C.ptr(indices), m, n,
                                                  rows.stride(0) if m > 1 else n, int(take_min),
                                                  _C.dtype_code(rows), _C.stream_ptr(tensor.device)),
                     "mdy_rowwise_extreme")
    values, indices = values.reshape(lead), indices.reshape(lead)
    if keepdim:
        values, indices = values.unsqueeze(axis), indices.unsqueeze(axis)
    return VALUES_INDICES(values, indices, "triton_min" if take_min else "triton_max")


def triton_max(tensor, axis=-1, keepdim=False):
    return _extreme(tensor, axis, keepdim, take_min=False)


def triton_min(tensor, axis=-1, keepdim=False):
    return _extreme(tensor, axis, keepdim, take_min=True)

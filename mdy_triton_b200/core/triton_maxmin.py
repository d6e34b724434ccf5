"""``triton_max`` / ``triton_min``: row-wise max / min with indices.

The reference exports these from ``mdy_triton/core/__init__.py:6`` (kernels in
``core/triton_maxmin.py``) but no patch module uses them; they are kept importable and delegate to
``torch.max`` / ``torch.min`` — they are not part of the accelerated path.
"""
import torch


def triton_max(x, dim=-1, keepdim=False):
    return torch.max(x, dim=dim, keepdim=keepdim)


def triton_min(x, dim=-1, keepdim=False):
    return torch.min(x, dim=dim, keepdim=keepdim)

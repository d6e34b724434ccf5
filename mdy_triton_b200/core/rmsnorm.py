"""RMSNorm operator: ``triton_rmsnorm(hidden_state, weight, eps)``.

Drop-in for the reference operator ``mdy_triton/core/rmsnorm.py:53-90`` (``_TritronRMSNorm`` /
``triton_rmsnorm``); the name keeps the reference's ``triton_`` prefix although the kernels behind it
are the sm_100a CUDA kernels of ``csrc/rmsnorm.cu``.
"""
from __future__ import annotations

import torch

from .. import _C


def _rows(t: torch.Tensor, n: int) -> torch.Tensor:
    """View ``t`` as [M, n] with unit inner stride (copy only if unavoidable)."""
    t2 = t.reshape(-1, n)
    if t2.stride(-1) != 1 or (t2.shape[0] > 1 and t2.stride(0) < n):
        t2 = t2.contiguous()
    return t2


class _TritronRMSNorm(torch.autograd.Function):
    """y = x / sqrt(mean(x^2) + eps) * weight (float32 math, output in x's dtype).

    Follows ``mdy_triton/core/rmsnorm.py:56-88``: saves the flattened input, the weight and one
    float32 statistic per row (here 1/rms instead of rms), returns ``dw`` in the weight's dtype.
    """

    @staticmethod
    def forward(ctx, hidden_state, weight, eps):
        dev = _C.require_cuda(hidden_state, weight)
        shape = hidden_state.shape
        n = shape[-1]
        x = _rows(hidden_state, n)
        m = x.shape[0]
        w = weight if weight.is_contiguous() else weight.contiguous()
        y = torch.empty(shape, dtype=hidden_state.dtype, device=dev)
        rstd = torch.empty(m, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _C.check(_C.lib().mdy_rmsnorm_fwd(_C.ptr(x), _C.ptr(w), _C.ptr(y), _C.ptr(rstd), m, n,
                                              x.stride(0) if m > 1 else n, n, float(eps),
                                              _C.dtype_code(x), _C.dtype_code(w), _C.stream_ptr(dev)),
                     "mdy_rmsnorm_fwd")
        ctx.save_for_backward(x, w, rstd)
        ctx.input_shape = shape
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        dev = x.device
        m, n = x.shape
        dy2 = _rows(dy, n)
        if dy2.dtype != x.dtype:
            dy2 = dy2.to(x.dtype)
        dx = torch.empty((m, n), dtype=x.dtype, device=dev)
        dw = torch.empty_like(w)
        lib = _C.lib()
        code = _C.dtype_code(x)
        with torch.cuda.device(dev):
            rows = lib.mdy_rmsnorm_bwd_partial_rows(m, n, code)
            partial = torch.empty((rows, n), dtype=torch.float32, device=dev)
            _C.check(lib.mdy_rmsnorm_bwd(_C.ptr(dy2), _C.ptr(x), _C.ptr(w), _C.ptr(rstd), _C.ptr(dx),
                                         _C.ptr(dw), _C.ptr(partial), m, n,
                                         dy2.stride(0) if m > 1 else n, x.stride(0) if m > 1 else n, n,
                                         code, _C.dtype_code(w), _C.stream_ptr(dev)),
                     "mdy_rmsnorm_bwd")
        return dx.view(ctx.input_shape), dw, None


triton_rmsnorm = _TritronRMSNorm.apply

"""Fused residual-add + RMSNorm: ``triton_fused_add_norm(x, residual, weight, eps) -> (y, new_residual)``.

Drop-in for ``mdy_triton/core/fused_add_norm.py:59-99`` (``_TritronFusedAddRMSNorm``).  The backward
follows the mathematics for every hidden size; the reference launch
(``fused_add_norm.py:85``, ``BLOCK_N = min(128, ...)`` without a column loop) is only correct up to
128 columns.
"""
from __future__ import annotations

import torch

from .. import _C


class _TritronFusedAddRMSNorm(torch.autograd.Function):
    """new_residual = x + residual; y = rmsnorm(new_residual) * weight.

    The sum is formed in float32 and normalised before it is rounded to the I/O dtype
    (``fused_add_norm.py:14-22``).  Backward returns ONE tensor as the gradient of both ``x`` and
    ``residual`` (the reference writes the same values to two buffers, ``:51-52``).
    """

    @staticmethod
    def forward(ctx, hidden_state, old_residual, weight, eps):
        dev = _C.require_cuda(hidden_state, old_residual, weight)
        if hidden_state.shape != old_residual.shape or hidden_state.dtype != old_residual.dtype:
            raise ValueError("hidden_state and residual must have the same shape and dtype")
        shape = hidden_state.shape
        n = shape[-1]
        x = hidden_state.contiguous().view(-1, n)
        r = old_residual.contiguous().view(-1, n)
        m = x.shape[0]
        w = weight if weight.is_contiguous() else weight.contiguous()
        y = torch.empty((m, n), dtype=x.dtype, device=dev)
        new_res = torch.empty((m, n), dtype=x.dtype, device=dev)
        rstd = torch.empty(m, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _C.check(_C.lib().mdy_add_rmsnorm_fwd(_C.ptr(x), _C.ptr(r), _C.ptr(w), _C.ptr(y),
                                                  _C.ptr(new_res), _C.ptr(rstd), m, n, n, float(eps),
                                                  _C.dtype_code(x), _C.dtype_code(w),
                                                  _C.stream_ptr(dev)),
                     "mdy_add_rmsnorm_fwd")
        new_res_out = new_res.view(shape)
        ctx.save_for_backward(new_res_out, w, rstd)
        ctx.input_shape = shape
        ctx.set_materialize_grads(False)
        return y.view(shape), new_res_out

    @staticmethod
    def backward(ctx, dy, dnew_res, *args):
        new_res, w, rstd = ctx.saved_tensors
        dev = new_res.device
        shape = ctx.input_shape
        n = shape[-1]
        new_res = new_res.view(-1, n)
        m = new_res.shape[0]
        lib = _C.lib()
        code = _C.dtype_code(new_res)
        if dy is None:
            # y was not used downstream: only the residual path carries gradient
            dw = torch.zeros_like(w)
            return dnew_res, dnew_res, dw, None
        dy2 = dy.to(new_res.dtype).contiguous().view(-1, n)
        dn2 = None if dnew_res is None else dnew_res.to(new_res.dtype).contiguous().view(-1, n)
        dx = torch.empty((m, n), dtype=new_res.dtype, device=dev)
        dw = torch.empty_like(w)
        with torch.cuda.device(dev):
            rows = lib.mdy_rmsnorm_bwd_partial_rows(m, n, code)
            partial = torch.empty((rows, n), dtype=torch.float32, device=dev)
            _C.check(lib.mdy_add_rmsnorm_bwd(_C.ptr(dy2), _C.ptr(dn2), _C.ptr(new_res), _C.ptr(w),
                                             _C.ptr(rstd), _C.ptr(dx), _C.ptr(dw), _C.ptr(partial), m, n,
                                             n, code, _C.dtype_code(w), _C.stream_ptr(dev)),
                     "mdy_add_rmsnorm_bwd")
        dx = dx.view(shape)
        return dx, dx, dw, None


triton_fused_add_norm = _TritronFusedAddRMSNorm.apply

"""SwiGLU operators: ``triton_fused_up_gate_silu(up, gate)`` and
``triton_fused_up_gate_silu_no_split(x, order='up-gate')``.

Drop-ins for ``mdy_triton/core/fused_silu.py:44-98`` (``_FusedSiLU_Unsloth``) and ``:170-234``
(``_FusedSiLUNoSplit``).  Both run on the same two CUDA kernels (``csrc/swiglu.cu``), which take a row
stride per tensor.
"""
from __future__ import annotations

import torch

from .. import _C


def _as_rows(t: torch.Tensor, n: int) -> torch.Tensor:
    """[.., n] -> [M, n] with unit inner stride and a usable row stride (copies only if needed)."""
    if t.dim() == 2 and t.stride(1) == 1 and (t.shape[0] <= 1 or t.stride(0) >= n):
        return t
    if t.is_contiguous():
        return t.view(-1, n)
    return t.reshape(-1, n).contiguous()


def _rs(t: torch.Tensor, n: int) -> int:
    return t.stride(0) if t.shape[0] > 1 else n


def _fwd(up2, gate2, y2, m, n):
    dev = up2.device
    with torch.cuda.device(dev):
        _C.check(_C.lib().mdy_swiglu_fwd(_C.ptr(up2), _C.ptr(gate2), _C.ptr(y2), m, n, _rs(up2, n),
                                         _rs(gate2, n), _rs(y2, n), _C.dtype_code(up2),
                                         _C.stream_ptr(dev)), "mdy_swiglu_fwd")


def _bwd(dy2, up2, gate2, dup2, dgate2, m, n):
    dev = up2.device
    with torch.cuda.device(dev):
        _C.check(_C.lib().mdy_swiglu_bwd(_C.ptr(dy2), _C.ptr(up2), _C.ptr(gate2), _C.ptr(dup2),
                                         _C.ptr(dgate2), m, n, _rs(dy2, n), _rs(up2, n), _rs(gate2, n),
                                         _rs(dup2, n), _rs(dgate2, n), _C.dtype_code(up2),
                                         _C.stream_ptr(dev)), "mdy_swiglu_bwd")


class _FusedSiLU_Unsloth(torch.autograd.Function):
    """y = up * silu(gate) for separate ``up`` and ``gate`` tensors of equal shape
    (``fused_silu.py:46-98``; argument order is (up, gate))."""

    @staticmethod
    def forward(ctx, up, gate):
        _C.require_cuda(up, gate)
        if up.shape != gate.shape or up.dtype != gate.dtype:
            raise ValueError("up and gate must have the same shape and dtype")
        n = up.shape[-1]
        up2, gate2 = _as_rows(up, n), _as_rows(gate, n)
        m = up2.shape[0]
        y = torch.empty(up.shape, dtype=up.dtype, device=up.device)
        _fwd(up2, gate2, y.view(-1, n), m, n)
        ctx.save_for_backward(up2, gate2)
        ctx.out_shape = up.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        up2, gate2 = ctx.saved_tensors
        m, n = up2.shape
        dy2 = _as_rows(dy.to(up2.dtype), n)
        dup = torch.empty(ctx.out_shape, dtype=up2.dtype, device=up2.device)
        dgate = torch.empty(ctx.out_shape, dtype=up2.dtype, device=up2.device)
        _bwd(dy2, up2, gate2, dup.view(-1, n), dgate.view(-1, n), m, n)
        return dup, dgate


class _FusedSiLUNoSplit(torch.autograd.Function):
    """y = up * silu(gate) where ``x = [up | gate]`` ('up-gate') or ``[gate | up]`` ('gate-up') along
    the last dimension (``fused_silu.py:170-231``)."""

    @staticmethod
    def forward(ctx, x, order="up-gate"):
        assert order in ["up-gate", "gate-up"], "please indicate the order of input, up-gate or gate-up"
        _C.require_cuda(x)
        shape = x.shape
        n2 = shape[-1]
        if n2 % 2:
            raise ValueError("last dimension must be even")
        n = n2 // 2
        x2 = _as_rows(x, n2)
        m = x2.shape[0]
        up2, gate2 = (x2[:, :n], x2[:, n:]) if order == "up-gate" else (x2[:, n:], x2[:, :n])
        y = torch.empty(*shape[:-1], n, dtype=x.dtype, device=x.device)
        _fwd(up2, gate2, y.view(-1, n), m, n)
        ctx.save_for_backward(x2)
        ctx.order = order
        ctx.in_shape = shape
        return y

    @staticmethod
    def backward(ctx, dy):
        (x2,) = ctx.saved_tensors
        m, n2 = x2.shape
        n = n2 // 2
        up2, gate2 = (x2[:, :n], x2[:, n:]) if ctx.order == "up-gate" else (x2[:, n:], x2[:, :n])
        dy2 = _as_rows(dy.to(x2.dtype), n)
        dx = torch.empty((m, n2), dtype=x2.dtype, device=x2.device)
        dup2, dgate2 = (dx[:, :n], dx[:, n:]) if ctx.order == "up-gate" else (dx[:, n:], dx[:, :n])
        _bwd(dy2, up2, gate2, dup2, dgate2, m, n)
        return dx.view(ctx.in_shape), None


triton_fused_up_gate_silu = _FusedSiLU_Unsloth.apply
triton_fused_up_gate_silu_no_split = _FusedSiLUNoSplit.apply

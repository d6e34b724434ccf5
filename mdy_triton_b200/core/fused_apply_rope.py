"""Fused rotary embedding on q and k: ``fused_apply_rope(q, k, cos, sin) -> (q, k)`` (in place).

Drop-in for ``mdy_triton/core/fused_apply_rope.py:92-140`` (``_FusedApplyRope``); it is assigned to
``modeling_<model>.apply_rotary_pos_emb`` by the patch modules, so it also accepts the optional
``position_ids`` / ``unsqueeze_dim`` arguments HuggingFace passes to that function.
"""
from __future__ import annotations

import torch

from .. import _C


def _bhl_strides(t: torch.Tensor):
    return t.stride(0), t.stride(1), t.stride(2)


def _launch(q_in, q_out, k_in, k_out, cos, sin, backward: bool):
    dev = q_in.device
    b, qh, l, d = q_in.shape
    kh = k_in.shape[1]
    with torch.cuda.device(dev):
        _C.check(_C.lib().mdy_rope(_C.ptr(q_in), _C.ptr(q_out), _C.ptr(k_in), _C.ptr(k_out), _C.ptr(cos),
                                   _C.ptr(sin), b, l, qh, kh, d, cos.shape[0],
                                   *_bhl_strides(q_in), *_bhl_strides(q_out),
                                   *_bhl_strides(k_in), *_bhl_strides(k_out),
                                   1 if backward else 0, _C.dtype_code(q_in), _C.stream_ptr(dev)),
                 "mdy_rope")


class _FusedApplyRope(torch.autograd.Function):
    """Rotate-half RoPE on q ``[B, QH, L, D]`` and k ``[B, KH, L, D]`` (logical shapes, any batch/head/
    position strides, unit stride on D) in one launch, writing the result back into q and k.

    Like the reference (``fused_apply_rope.py:94-125``) the inputs are modified in place and returned;
    cos/sin are ``[B or 1, L, D]``.  Backward (``:128-138``) applies the transposed rotation to the
    incoming gradients; it writes them to fresh ``[B, L, H, D]``-contiguous buffers, the layout the
    q/k projections' backward consumes without a copy.
    """

    @staticmethod
    def forward(ctx, q, k, cos, sin):
        _C.require_cuda(q, k, cos, sin)
        if q.dim() != 4 or k.dim() != 4:
            raise ValueError("q and k must be [batch, heads, seq, head_dim]")
        if q.stride(-1) != 1 or k.stride(-1) != 1:
            raise ValueError("q and k must have unit stride on head_dim")
        if q.dtype != k.dtype:
            raise ValueError("q and k must share a dtype")
        b, qh, l, d = q.shape
        if k.shape[0] != b or k.shape[2] != l or k.shape[3] != d:
            raise ValueError("q and k disagree on batch, seq or head_dim")
        if cos.dim() == 2:
            cos, sin = cos.unsqueeze(0), sin.unsqueeze(0)
        rd = cos.shape[-1]
        if (cos.shape[-2] != l or rd > d or rd % 2 or rd == 0 or cos.shape != sin.shape
                or cos.shape[0] not in (1, b)):
            raise ValueError(f"cos/sin must be [{b} or 1, {l}, rotary_dim <= {d}], got {tuple(cos.shape)}")
        cos = cos.to(q.dtype).contiguous()
        sin = sin.to(q.dtype).contiguous()
        # Partial rotary embedding (HuggingFace Phi3 / GLM with partial_rotary_factor < 1: rotary_dim =
        # cos.shape[-1]): only the first rotary_dim columns of every head are rotated, the rest pass through.
        # The kernel takes the head stride separately from the rotated width, so it runs on a view.
        qv, kv = (q, k) if rd == d else (q[..., :rd], k[..., :rd])
        _launch(qv, qv, kv, kv, cos, sin, backward=False)
        ctx.save_for_backward(cos, sin)
        return q, k

    @staticmethod
    def backward(ctx, dq, dk):
        cos, sin = ctx.saved_tensors
        if dq.stride(-1) != 1:
            dq = dq.contiguous()
        if dk.stride(-1) != 1:
            dk = dk.contiguous()
        if dq.dtype != cos.dtype:
            dq = dq.to(cos.dtype)
        if dk.dtype != cos.dtype:
            dk = dk.to(cos.dtype)
        b, qh, l, d = dq.shape
        kh = dk.shape[1]
        dq_out = torch.empty((b, l, qh, d), dtype=dq.dtype, device=dq.device).transpose(1, 2)
        dk_out = torch.empty((b, l, kh, d), dtype=dk.dtype, device=dk.device).transpose(1, 2)
        rd = cos.shape[-1]
        if rd == d:
            _launch(dq, dq_out, dk, dk_out, cos, sin, backward=True)
        else:
            _launch(dq[..., :rd], dq_out[..., :rd], dk[..., :rd], dk_out[..., :rd], cos, sin, backward=True)
            dq_out[..., rd:].copy_(dq[..., rd:])
            dk_out[..., rd:].copy_(dk[..., rd:])
        return dq_out, dk_out, None, None


def fused_apply_rope(q, k, cos, sin, position_ids=None, unsqueeze_dim=1):
    """``apply_rotary_pos_emb`` replacement.  ``position_ids`` is accepted and ignored (cos/sin are
    already gathered per position); ``unsqueeze_dim=2`` means q/k are ``[B, L, H, D]``."""
    if unsqueeze_dim == 2:
        q2, k2 = _FusedApplyRope.apply(q.transpose(1, 2), k.transpose(1, 2), cos, sin)
        return q2.transpose(1, 2), k2.transpose(1, 2)
    return _FusedApplyRope.apply(q, k, cos, sin)

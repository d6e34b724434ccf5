"""Large-vocab cross-entropy: ``triton_entropy_loss`` / ``fast_cross_entropy_loss`` and the per-row
``_FastCrossEntropyLoss`` (the file name keeps the reference's spelling).

Drop-in for ``mdy_triton/core/cross_entyopy_loss.py:82-149``.  The patch modules of the reference call
``fast_cross_entropy_loss(logits, labels, n_items=...)`` (``replace_kernel/llama.py:171-172``), a name
the reference file no longer defines; it is provided here with the same meaning as
``triton_entropy_loss``.

Two execution paths:
  * per-row API (``_FastCrossEntropyLoss.apply``): forward sweep writes ``losses``/``lse``, backward
    sweep writes ``dlogits`` from an arbitrary per-row upstream gradient — same contract as the reference.
  * scalar-loss API (``triton_entropy_loss`` / ``fast_cross_entropy_loss``) with gradients enabled, for
    bfloat16 and float32 logits: the gradient of ``sum(losses) / n_items`` w.r.t. each row is the constant
    ``1 / n_items``, known before the kernel starts, so ONE kernel computes the loss and writes ``dlogits``
    in a single pass over the logits; backward only rescales if the incoming gradient is not 1.  That
    gradient buffer can be handed out once: a second backward through the same loss raises.
    float16 logits and ``inplace=True`` take the per-row path instead: with a loss scaler the product
    ``dloss * (softmax - onehot)`` has to be formed in float32 before it is rounded to float16 (the
    unscaled ``(softmax - onehot) / n_items`` of a rare token underflows there), and in-place callers expect
    their logits to stay intact until backward, as in the reference.
"""
from __future__ import annotations

import os

import torch

from .. import _C

IGNORE_INDEX = -100

# When True, the scalar-loss API overwrites ``logits`` with ``dlogits`` (as the reference does with
# ``inplace=True``) instead of allocating a gradient buffer.  Per call: ``inplace=`` argument.
INPLACE_DEFAULT = os.environ.get("MDY_CE_INPLACE", "0") == "1"


def _flat(logits: torch.Tensor, labels: torch.Tensor):
    if not logits.is_contiguous():
        raise ValueError("logits must be contiguous")  # reference asserts the same (:86)
    v = logits.shape[-1]
    lg = logits.view(-1, v)
    lb = labels.reshape(-1)
    if lb.dtype != torch.int64:
        lb = lb.to(torch.int64)
    lb = lb.contiguous()
    if lb.shape[0] != lg.shape[0]:
        raise ValueError(f"labels have {lb.shape[0]} entries for {lg.shape[0]} rows of logits")
    return lg, lb


def ce_forward_rows(lg, lb, vocab_start=0, split=False):
    """losses[M], lse[M] (float32) of logits ``lg`` [M, V]; see ``mdy_ce_fwd``."""
    dev = _C.require_cuda(lg, lb)
    m, v = lg.shape
    losses = torch.empty(m, dtype=torch.float32, device=dev)
    lse = torch.empty(m, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _C.check(_C.lib().mdy_ce_fwd(_C.ptr(lg), _C.ptr(lb), _C.ptr(losses), _C.ptr(lse), m, v,
                                     lg.stride(0) if m > 1 else v, vocab_start, 1 if split else 0,
                                     _C.dtype_code(lg), _C.stream_ptr(dev)), "mdy_ce_fwd")
    return losses, lse


def ce_backward_rows(dlosses, lg, lb, lse, dlogits, vocab_start=0):
    """dlogits[M, V] from per-row upstream gradients; ignored rows are zero-filled.  See ``mdy_ce_bwd``."""
    dev = lg.device
    m, v = lg.shape
    dl = dlosses.reshape(-1) if dlosses.numel() == m else dlosses.expand(m)
    if dl.dtype not in _C.DTYPE_CODE:
        dl = dl.float()
    with torch.cuda.device(dev):
        _C.check(_C.lib().mdy_ce_bwd(_C.ptr(dl), dl.stride(0) if m > 1 else 1, _C.dtype_code(dl),
                                     _C.ptr(lg), _C.ptr(dlogits), _C.ptr(lb), _C.ptr(lse), m, v,
                                     lg.stride(0) if m > 1 else v, vocab_start, 1, _C.dtype_code(lg),
                                     _C.stream_ptr(dev)), "mdy_ce_bwd")
    return dlogits


class _FastCrossEntropyLoss(torch.autograd.Function):
    """Per-row losses ``lse - logit[label]`` (0 where label == -100), shape ``logits.shape[:-1]``.

    Same contract as ``cross_entyopy_loss.py:85-142``: ``inplace=True`` makes backward write the
    gradient into the logits' own storage.  Without ``inplace`` the gradient buffer is allocated
    uninitialised and the kernel zero-fills ignored rows (the reference pays a ``zeros_like`` pass).
    """

    @staticmethod
    def forward(ctx, logits, labels, inplace=False):
        lg, lb = _flat(logits, labels)
        losses, lse = ce_forward_rows(lg, lb)
        ctx.save_for_backward(lg, lb, lse)
        ctx.inplace = bool(inplace)
        ctx.input_shape = logits.shape
        return losses.view(logits.shape[:-1])

    @staticmethod
    def backward(ctx, dlosses):
        lg, lb, lse = ctx.saved_tensors
        dlogits = lg if ctx.inplace else torch.empty_like(lg)
        ce_backward_rows(dlosses, lg, lb, lse, dlogits)
        return dlogits.view(ctx.input_shape), None, None


class _FusedLossAndGrad(torch.autograd.Function):
    """Scalar ``sum(losses) / n_items`` whose forward already writes ``dlogits`` (one pass over HBM)."""

    @staticmethod
    def forward(ctx, logits, labels, n_items, inplace):
        lg, lb = _flat(logits, labels)
        dev = _C.require_cuda(lg, lb)
        m, v = lg.shape
        if n_items is None:
            n = torch.count_nonzero(lb != IGNORE_INDEX).to(torch.float32)
        else:
            n = torch.as_tensor(n_items, device=dev).to(torch.float32)
        inv = n.reciprocal().reshape(1)
        losses = torch.empty(m, dtype=torch.float32, device=dev)
        lse = torch.empty(m, dtype=torch.float32, device=dev)
        dlogits = lg if inplace else torch.empty_like(lg)
        with torch.cuda.device(dev):
            _C.check(_C.lib().mdy_ce_fused(_C.ptr(lg), _C.ptr(dlogits), _C.ptr(lb), _C.ptr(losses),
                                           _C.ptr(lse), _C.ptr(inv), 1.0, m, v,
                                           lg.stride(0) if m > 1 else v, _C.dtype_code(lg),
                                           _C.stream_ptr(dev)), "mdy_ce_fused")
        ctx.save_for_backward(dlogits)
        ctx.input_shape = logits.shape
        ctx.consumed = False
        return losses.sum() * inv[0]

    @staticmethod
    def backward(ctx, dloss):
        if ctx.consumed:
            raise RuntimeError("the one-pass cross-entropy hands its gradient buffer out once: a second backward "
                               "through the same loss would rescale the gradient it already returned; recompute the "
                               "loss, or use _FastCrossEntropyLoss.apply for a graph that is walked twice")
        ctx.consumed = True
        (dlogits,) = ctx.saved_tensors
        dev = dlogits.device
        g = dloss.detach().to(device=dev, dtype=torch.float32).reshape(1).contiguous()
        with torch.cuda.device(dev):
            # no memory traffic when the upstream gradient is exactly 1 (the usual case)
            _C.check(_C.lib().mdy_scale_inplace(_C.ptr(dlogits), dlogits.numel(), _C.ptr(g),
                                                _C.dtype_code(dlogits), _C.stream_ptr(dev)),
                     "mdy_scale_inplace")
        return dlogits.view(ctx.input_shape), None, None, None


def triton_entropy_loss(logits, labels, num_items_in_batch=None, inplace=None):
    """Mean cross-entropy over rows whose label is not -100: ``sum(losses) / num_items_in_batch``
    (``cross_entyopy_loss.py:145-149``); ``num_items_in_batch`` defaults to the count of such rows."""
    if inplace is None:
        inplace = INPLACE_DEFAULT
    if torch.is_grad_enabled() and logits.requires_grad:
        if logits.dtype != torch.float16 and not inplace:
            return _FusedLossAndGrad.apply(logits, labels, num_items_in_batch, False)
        losses = _FastCrossEntropyLoss.apply(logits, labels, bool(inplace))
        if num_items_in_batch is None:
            num_items_in_batch = torch.count_nonzero(labels != IGNORE_INDEX)
        return losses.sum() / num_items_in_batch
    lg, lb = _flat(logits, labels)
    losses, _ = ce_forward_rows(lg, lb)
    if num_items_in_batch is None:
        num_items_in_batch = torch.count_nonzero(lb != IGNORE_INDEX)
    return losses.sum() / num_items_in_batch


def fast_cross_entropy_loss(logits, labels, n_items=None):
    """Name the patch modules import (``replace_kernel/llama.py:6,171-172``):
    ``logits`` [B, L, V], ``labels`` [B, L] -> scalar ``sum / n_items``."""
    return triton_entropy_loss(logits, labels, n_items)

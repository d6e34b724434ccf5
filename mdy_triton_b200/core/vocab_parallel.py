"""Vocab-parallel cross-entropy: every rank holds ``logits[..., r*V/g:(r+1)*V/g]`` and all labels.

Restates the tensor-parallel branch of the reference's loss
(``triton_kernels/cross_entropy/test_ce.py:110-166``; the same code is dead in
``mdy_triton/core/cross_entyopy_loss.py:109-117`` because ``tp_size`` is hard-coded to 1):
local sweep -> exchange of per-row statistics -> global lse and loss -> local gradient sweep with the
global lse.  The exchange is ONE ``all_gather_into_tensor`` of a float32 ``[2, M]`` tensor per rank
(local lse, and ``-logit[label]`` on the rank that owns the label) on the given process group; the
reference uses an all-gather plus an all-reduce on the default group.  Backward needs no collective.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import _C
from . import cross_entyopy_loss as _ce


def _local_forward(lg, lb, vocab_start, stats):
    """Fill stats[0] = local lse, stats[1] = -logit[label] if owned else 0 (float32 [2, M])."""
    dev = _C.require_cuda(lg, lb, stats)
    m, v = lg.shape
    with torch.cuda.device(dev):
        _C.check(_C.lib().mdy_ce_fwd(_C.ptr(lg), _C.ptr(lb), _C.ptr(stats[1]), _C.ptr(stats[0]), m, v,
                                     lg.stride(0) if m > 1 else v, vocab_start, 1, _C.dtype_code(lg),
                                     _C.stream_ptr(dev)), "mdy_ce_fwd")


def _combine(gathered, lb):
    """gathered float32 [tp, 2, M] -> (losses[M], lse[M])."""
    dev = gathered.device
    tp, _, m = gathered.shape
    losses = torch.empty(m, dtype=torch.float32, device=dev)
    lse = torch.empty(m, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _C.check(_C.lib().mdy_ce_vp_combine(_C.ptr(gathered), _C.ptr(lb), _C.ptr(losses), _C.ptr(lse), tp,
                                            m, _C.stream_ptr(dev)), "mdy_ce_vp_combine")
    return losses, lse


def _local_backward(dlosses, lg, lb, lse, dlogits, vocab_start):
    return _ce.ce_backward_rows(dlosses, lg, lb, lse, dlogits, vocab_start)


class _VocabParallelCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, group, inplace):
        lg, lb = _ce._flat(logits, labels)
        tp = dist.get_world_size(group)
        rank = dist.get_rank(group)
        m, v = lg.shape
        vocab_start = v * rank
        # ignored rows must carry neutral statistics on every rank (-inf lse would also do; 0/0 is
        # what the local kernel writes and the combine step masks them by label)
        stats = torch.empty((2, m), dtype=torch.float32, device=lg.device)
        _local_forward(lg, lb, vocab_start, stats)
        gathered = torch.empty((tp, 2, m), dtype=torch.float32, device=lg.device)
        dist.all_gather_into_tensor(gathered.view(-1), stats.view(-1), group=group)
        losses, lse = _combine(gathered, lb)
        ctx.save_for_backward(lg, lb, lse)
        ctx.inplace = bool(inplace)
        ctx.vocab_start = vocab_start
        ctx.input_shape = logits.shape
        return losses.view(logits.shape[:-1])

    @staticmethod
    def backward(ctx, dlosses):
        lg, lb, lse = ctx.saved_tensors
        dlogits = lg if ctx.inplace else torch.empty_like(lg)
        _local_backward(dlosses, lg, lb, lse, dlogits, ctx.vocab_start)
        return dlogits.view(ctx.input_shape), None, None, None


def vocab_parallel_cross_entropy(logits, labels, group=None, inplace=False):
    """Per-row losses for vocab-sharded ``logits`` [..., V/g] and replicated ``labels`` [...]
    (global vocabulary ids, -100 = ignored).  Identical on every rank of ``group``."""
    return _VocabParallelCrossEntropy.apply(logits, labels, group, inplace)


def vocab_parallel_entropy_loss(logits, labels, num_items_in_batch=None, group=None, inplace=False):
    """Scalar ``sum(losses) / num_items_in_batch`` on vocab-sharded logits (same on every rank)."""
    losses = vocab_parallel_cross_entropy(logits, labels, group, inplace)
    if num_items_in_batch is None:
        num_items_in_batch = torch.count_nonzero(labels != _ce.IGNORE_INDEX)
    return losses.sum() / num_items_in_batch

"""Vocab-parallel cross-entropy: every rank holds ``logits[..., r*V/g:(r+1)*V/g]`` and all labels.

Restates the tensor-parallel branch of the reference's loss
(``triton_kernels/cross_entropy/test_ce.py:110-166``; the same code is dead in
``mdy_triton/core/cross_entyopy_loss.py:109-117`` because ``tp_size`` is hard-coded to 1):
local sweep -> exchange of per-row statistics -> global lse and loss -> local gradient sweep with the
global lse.  The exchange is ONE ``all_gather_into_tensor`` of a float32 ``[2, M]`` tensor per rank
(local lse, and ``-logit[label]`` on the rank that owns the label) on the given process group; the
reference uses an all-gather plus an all-reduce on the default group.  Backward needs no collective.

``vocab_parallel_entropy_loss`` (the scalar loss, whose per-row upstream gradient ``1 / n_items`` is known
before the kernel starts) can go further when it is given a :class:`PeerExchange`: ONE kernel per GPU
computes the statistics, exchanges them by storing straight into the peers' memory over NVLink, and writes
the gradient from the row slices it still holds in shared memory (``mdy_ce_vp_fused``) — the shard is read
once and written once and there is no NCCL call on the path.
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


class PeerExchange:
    """Exchange buffers for the one-kernel path: one buffer per rank of ``group``, allocated by the
    library (a peer has to be able to map it), made known to the other ranks through CUDA IPC handles that
    travel over ``group`` once, here.  ``max_rows`` bounds the rows of a call; ``shard_cols`` and ``dtype``
    fix the geometry.  Create it once, outside the training loop (it allocates and synchronises), and pass
    it to :func:`vocab_parallel_entropy_loss`; every rank must then make the same calls in the same order.
    With ``group=None`` and no initialised process group it serves a single rank."""

    def __init__(self, max_rows, shard_cols, dtype, device, group=None):
        import ctypes
        self.group = group
        self.device = torch.device(device)
        self.tp = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.max_rows, self.shard_cols, self.dtype = int(max_rows), int(shard_cols), dtype
        lib = _C.lib()
        nbytes = lib.mdy_ce_vp_exchange_bytes(self.max_rows, self.shard_cols, self.tp, _C.DTYPE_CODE[dtype])
        if nbytes < 0:
            raise ValueError(f"no one-kernel geometry for shards of {shard_cols} columns over {self.tp} ranks: "
                             f"{_C.status_string(nbytes)}")
        self.epoch = 0
        self._own = ctypes.c_void_p()
        self._opened = []
        handle = ctypes.create_string_buffer(64)
        with torch.cuda.device(self.device):
            _C.check(lib.mdy_peer_buffer_create(nbytes, ctypes.byref(self._own), handle), "mdy_peer_buffer_create")
            ptrs = [None] * self.tp
            ptrs[self.rank] = self._own.value
            if self.tp > 1:
                handles = [None] * self.tp
                dist.all_gather_object(handles, handle.raw, group=group)
                for r, h in enumerate(handles):
                    if r == self.rank:
                        continue
                    p = ctypes.c_void_p()
                    _C.check(lib.mdy_peer_buffer_open(ctypes.create_string_buffer(h, 64), ctypes.byref(p)),
                             f"mdy_peer_buffer_open(rank {r})")
                    self._opened.append(p.value)
                    ptrs[r] = p.value
                dist.barrier(group=group)   # nobody launches before every rank has mapped every buffer
        self.ptrs = (ctypes.c_void_p * self.tp)(*ptrs)

    def next_epoch(self):
        # wraps from the odd 0xFFFFFFFF to the even 2: consecutive launches always use different halves of the buffers
        self.epoch = self.epoch + 1 if self.epoch < 0xFFFFFFFF else 2
        return self.epoch

    def close(self):
        """Unmap the peers' buffers and free this rank's.  Call on every rank once no kernel uses them."""
        lib = _C.lib()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            for p in self._opened:
                lib.mdy_peer_buffer_close(p)
            self._opened = []
            if self.tp > 1 and dist.is_initialized():
                dist.barrier(group=self.group)   # a buffer is freed only after every peer has unmapped it
            if self._own.value:
                lib.mdy_peer_buffer_destroy(self._own)
                self._own.value = None


def fused_launcher(lg, lb, dlogits, inv_n, exchange: PeerExchange):
    """Prepare repeated launches of ``mdy_ce_vp_fused`` on fixed buffers (a training loop with static shapes,
    a benchmark): returns ``(launch, losses, lse)`` where ``launch()`` does nothing on the host but advance
    the epoch and make the C call on the current stream of the shard's device."""
    import ctypes
    dev = _C.require_cuda(lg, lb, dlogits)
    m, v = lg.shape
    if v != exchange.shard_cols or m > exchange.max_rows or lg.dtype != exchange.dtype:
        raise ValueError("the PeerExchange was created for another shard shape")
    losses = torch.empty(m, dtype=torch.float32, device=dev)
    lse = torch.empty(m, dtype=torch.float32, device=dev)
    one = lambda t: (ctypes.c_void_p * 1)(t.data_ptr())
    a_lg, a_dl, a_lo, a_ls = one(lg), one(dlogits), one(losses), one(lse)
    fn = _C.lib().mdy_ce_vp_fused
    p_lb, p_inv, stride, code = _C.ptr(lb), _C.ptr(inv_n), (lg.stride(0) if m > 1 else v), _C.dtype_code(lg)

    def launch():
        rc = fn(a_lg, a_dl, a_lo, a_ls, exchange.ptrs, p_lb, p_inv, 1.0, m, v, stride, exchange.tp, exchange.rank, 1,
                exchange.max_rows, exchange.next_epoch(), code, torch.cuda.current_stream(dev).cuda_stream)
        if rc != 0:
            _C.check(rc, "mdy_ce_vp_fused")
    return launch, losses, lse


def fused_loss_and_grad(lg, lb, dlogits, inv_n, exchange: PeerExchange):
    """One launch of ``mdy_ce_vp_fused`` for this rank's shard ``lg`` [M, Vs]: writes ``dlogits`` (may be
    ``lg``) scaled by ``inv_n`` (float32 device scalar) and returns (losses[M], lse[M])."""
    import ctypes
    dev = _C.require_cuda(lg, lb, dlogits)
    m, v = lg.shape
    if v != exchange.shard_cols or m > exchange.max_rows or lg.dtype != exchange.dtype:
        raise ValueError("the PeerExchange was created for another shard shape")
    losses = torch.empty(m, dtype=torch.float32, device=dev)
    lse = torch.empty(m, dtype=torch.float32, device=dev)
    one = lambda t: (ctypes.c_void_p * 1)(t.data_ptr())
    with torch.cuda.device(dev):
        _C.check(_C.lib().mdy_ce_vp_fused(one(lg), one(dlogits), one(losses), one(lse), exchange.ptrs, _C.ptr(lb),
                                          _C.ptr(inv_n), 1.0, m, v, lg.stride(0) if m > 1 else v, exchange.tp,
                                          exchange.rank, 1, exchange.max_rows, exchange.next_epoch(),
                                          _C.dtype_code(lg), _C.stream_ptr(dev)), "mdy_ce_vp_fused")
    return losses, lse


class _FusedVocabParallelLoss(torch.autograd.Function):
    """Scalar ``sum(losses) / n_items`` on vocab-sharded logits whose forward already wrote the gradient."""

    @staticmethod
    def forward(ctx, logits, labels, n_items, exchange, inplace):
        lg, lb = _ce._flat(logits, labels)
        dev = lg.device
        if n_items is None:
            n = torch.count_nonzero(lb != _ce.IGNORE_INDEX).to(torch.float32)
        else:
            n = torch.as_tensor(n_items, device=dev).to(torch.float32)
        inv = n.reciprocal().reshape(1)
        dlogits = lg if inplace else torch.empty_like(lg)
        losses, _ = fused_loss_and_grad(lg, lb, dlogits, inv, exchange)
        ctx.save_for_backward(dlogits)
        ctx.input_shape = logits.shape
        ctx.consumed = False
        return losses.sum() * inv[0]

    @staticmethod
    def backward(ctx, dloss):
        if ctx.consumed:
            raise RuntimeError("the one-kernel vocab-parallel loss hands its gradient buffer out once")
        ctx.consumed = True
        (dlogits,) = ctx.saved_tensors
        dev = dlogits.device
        g = dloss.detach().to(device=dev, dtype=torch.float32).reshape(1).contiguous()
        with torch.cuda.device(dev):
            _C.check(_C.lib().mdy_scale_inplace(_C.ptr(dlogits), dlogits.numel(), _C.ptr(g),
                                                _C.dtype_code(dlogits), _C.stream_ptr(dev)), "mdy_scale_inplace")
        return dlogits.view(ctx.input_shape), None, None, None, None


def vocab_parallel_cross_entropy(logits, labels, group=None, inplace=False):
    """Per-row losses for vocab-sharded ``logits`` [..., V/g] and replicated ``labels`` [...]
    (global vocabulary ids, -100 = ignored).  Identical on every rank of ``group``."""
    return _VocabParallelCrossEntropy.apply(logits, labels, group, inplace)


def vocab_parallel_entropy_loss(logits, labels, num_items_in_batch=None, group=None, inplace=False, exchange=None):
    """Scalar ``sum(losses) / num_items_in_batch`` on vocab-sharded logits (same on every rank).  With a
    :class:`PeerExchange` (and gradients enabled, logits not float16, not ``inplace``: in-place callers expect
    their logits intact until backward) the loss and the gradient come from one kernel per GPU that exchanges
    the row statistics through peer memory; otherwise from the sweep -> all-gather -> sweep path."""
    if (exchange is not None and torch.is_grad_enabled() and logits.requires_grad
            and logits.dtype != torch.float16 and not inplace):
        return _FusedVocabParallelLoss.apply(logits, labels, num_items_in_batch, exchange, False)
    losses = vocab_parallel_cross_entropy(logits, labels, group, inplace)
    if num_items_in_batch is None:
        num_items_in_batch = torch.count_nonzero(labels != _ce.IGNORE_INDEX)
    return losses.sum() / num_items_in_batch

"""Time the reference's own Triton kernels on the GPU at hand.  Test / benchmark infrastructure only.

Each operator is driven through the ``forward`` / ``backward`` static methods of the reference's
``torch.autograd.Function`` (its stock host code: output allocation, block-size choice, kernel launch,
the host-side ``dw.sum(0)``) with a stand-in context object, so forward and backward can be timed apart
with CUDA events on the current stream.  The kernels come from ``oracle/_ref`` through
``oracle/ref_loader.py`` (native mode: Triton's JIT, no interpreter).
"""
from __future__ import annotations

import statistics

import torch

from . import ref_loader as R


class _Ctx:
    """What the reference's forward/backward use of an autograd context: saved tensors and attributes."""
    needs_input_grad = (True, True, True, True)

    def save_for_backward(self, *tensors):
        self.saved_tensors = tensors

    def mark_dirty(self, *tensors):
        pass


def _time(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ms = []
    for _ in range(iters):
        if flush is not None:
            flush.fill_(1)
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        ms.append(e0.elapsed_time(e1))
    return statistics.median(ms)


def time_reference_ops(ops, iters=5, warmup=2, flush=False):
    """`ops`: an object holding one configuration's device tensors (bench.OpSet).  Returns
    {operator: {"fwd_ms", "bwd_ms", "ms"}} for the reference's kernels on those tensors.  In-place
    operators (RoPE; cross-entropy with inplace=True) work on scratch copies."""
    if not (R.available() and R.native()):
        raise RuntimeError("the reference kernels need their staged files and a CUDA device")
    cfg = ops.cfg
    buf = torch.empty(256 << 20, dtype=torch.uint8, device=ops.dev) if flush else None
    out = {}

    def pair(name, fwd, bwd):
        f = _time(fwd, iters, warmup, buf)
        b = _time(bwd, iters, warmup, buf)
        out[name] = {"fwd_ms": f, "bwd_ms": b, "ms": f + b}

    # RMSNorm / add+RMSNorm (core/rmsnorm.py:53-90, core/fused_add_norm.py:59-99)
    if cfg["norm"] == "add_rmsnorm":
        F = R.load("fused_add_norm")._TritronFusedAddRMSNorm
        ctx = _Ctx()
        pair("norm", lambda: F.forward(ctx, ops.x, ops.res, ops.w, cfg["eps"]),
             lambda: F.backward(ctx, ops.dy, ops.dnres))
        out["norm"]["note"] = "backward reads 128 of the columns only (its result is not the gradient); timed, not compared"
    else:
        F = R.load("rmsnorm")._TritronRMSNorm
        ctx = _Ctx()
        pair("norm", lambda: F.forward(ctx, ops.x, ops.w, cfg["eps"]), lambda: F.backward(ctx, ops.dy))
    # RoPE, in place on copies (core/fused_apply_rope.py:92-140)
    F = R.load("fused_apply_rope")._FusedApplyRope
    q, k, dq, dk = (t.clone() for t in (ops.q, ops.k, ops.dq, ops.dk))
    tr = lambda t: t.transpose(1, 2)
    ctx_r = _Ctx()
    pair("rope", lambda: F.forward(ctx_r, tr(q), tr(k), ops.cos, ops.sin), lambda: F.backward(ctx_r, tr(dq), tr(dk)))
    del q, k, dq, dk
    # SwiGLU (core/fused_silu.py:44-98)
    F = R.load("fused_silu")._FusedSiLU_Unsloth
    ctx_s = _Ctx()
    pair("swiglu", lambda: F.forward(ctx_s, ops.up, ops.gate), lambda: F.backward(ctx_s, ops.sdy))
    # cross-entropy (core/cross_entyopy_loss.py:82-142): as shipped (gradient in a zero-filled new tensor),
    # and in place (its fastest mode: three passes over the logits instead of four)
    F = R.load("cross_entyopy_loss")._FastCrossEntropyLoss
    M = ops.M
    dlosses = torch.full((M,), 1.0 / M, device=ops.dev)
    ctx_c = _Ctx()
    pair("cross_entropy", lambda: F.forward(ctx_c, ops.logits, ops.labels, False), lambda: F.backward(ctx_c, dlosses))
    work = ops.dlogits  # scratch of the same shape: the in-place mode overwrites its input
    work.copy_(ops.logits)
    ctx_i = _Ctx()
    pair("cross_entropy_inplace", lambda: F.forward(ctx_i, work, ops.labels, True), lambda: F.backward(ctx_i, dlosses))
    torch.cuda.empty_cache()
    return out

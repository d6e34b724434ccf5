"""Megatron-LM facing adapters on top of the same kernels (signature level: Megatron-LM itself is not
a dependency of this package).

``swiglu_impl(x, bias, fp8_input_store)`` follows ``triton_kernels/megatron_patchs/swiglu.py:138-139``
(fused projection in 'gate-up' order); ``vocab_parallel_cross_entropy(logits, labels)`` follows
``triton_kernels/megatron_patchs/cross_entropy_losss.py:139-140`` (per-token losses on vocab-sharded
logits, gradient written in place) with the tensor-parallel group passed explicitly.
"""
from __future__ import annotations

from .fused_silu import triton_fused_up_gate_silu_no_split
from .vocab_parallel import vocab_parallel_cross_entropy as _vp_ce


def swiglu_impl(x, bias=None, fp8_input_store=False):
    """SwiGLU on a fused ``[..., 2N]`` projection laid out ``[gate | up]``.  ``bias`` is added first when
    given; ``fp8_input_store`` (an activation-memory option of TransformerEngine) is accepted and ignored."""
    if bias is not None:
        x = x + bias
    return triton_fused_up_gate_silu_no_split(x, "gate-up")


def vocab_parallel_cross_entropy(vocab_parallel_logits, target, tp_group=None):
    """Per-token losses for logits sharded over ``tp_group`` along the vocabulary; the gradient reuses the
    logits' storage, as the reference adapter does."""
    return _vp_ce(vocab_parallel_logits, target, tp_group, True)

"""Operator API of the reference's ``mdy_triton.core`` (``core/__init__.py:1-6``), backed by the
sm_100a CUDA library."""
from .cross_entyopy_loss import fast_cross_entropy_loss, triton_entropy_loss, _FastCrossEntropyLoss
from .fused_add_norm import triton_fused_add_norm
from .fused_silu import triton_fused_up_gate_silu, triton_fused_up_gate_silu_no_split
from .fused_apply_rope import fused_apply_rope
from .rmsnorm import triton_rmsnorm
from .triton_maxmin import triton_min, triton_max
from .vocab_parallel import vocab_parallel_cross_entropy, vocab_parallel_entropy_loss

__all__ = [
    "fast_cross_entropy_loss", "triton_entropy_loss", "triton_fused_add_norm",
    "triton_fused_up_gate_silu", "triton_fused_up_gate_silu_no_split", "fused_apply_rope",
    "triton_rmsnorm", "triton_min", "triton_max", "vocab_parallel_cross_entropy",
    "vocab_parallel_entropy_loss",
]

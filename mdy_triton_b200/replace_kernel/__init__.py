"""``from mdy_triton.replace_kernel import *`` — importing this package swaps the RMSNorm, MLP,
decoder-layer and causal-LM forwards and ``apply_rotary_pos_emb`` of HuggingFace Llama, Qwen2, Qwen2-VL,
Mistral and Phi3 for the fused kernels (reference: mdy_triton/replace_kernel/__init__.py:1-5).  The swap is
process-wide and not reversible; it also affects models that were instantiated before the import.
"""
from .llama import trigger
from .qwen2 import trigger
from .qwen2_vl import trigger
from .mistral import trigger
from .phi3 import trigger
from ._common import residual_fusion_enabled, set_residual_fusion

__all__ = ["trigger", "set_residual_fusion", "residual_fusion_enabled"]

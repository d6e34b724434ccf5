"""Patch the GLM-4 modules with the fused kernels at import time (reference:
mdy_triton/replace_kernel/glm4.py).

The reference patches the remote-code ``modeling_chatglm`` it loads from a model directory on its author's
machine (glm4.py:13-15).  transformers ships the same network as ``transformers.models.glm`` (the
``glm-4-9b-chat-hf`` port), and that is what is patched here: RMSNorm, the MLP with its single
gate/up projection (no-split SwiGLU, 'gate-up' order as at glm4.py:29-35), the decoder layer with the
post-attention add fused into the norm (glm4.py:37-75) and the causal-LM loss.  RoPE stays stock, as in the
reference (glm4.py:5-6: GLM rotates interleaved pairs of half of each head).  Like the reference's package
``__init__`` (which lists five families, not this one), ``from mdy_triton.replace_kernel import *`` does not
import this module: ``import mdy_triton.replace_kernel.glm4`` applies it.
"""
import importlib

from ._common import mlp_forward_fused_proj, patch_family

module = importlib.import_module("transformers.models.glm.modeling_glm")
patch_family(module, "Glm", mlp=mlp_forward_fused_proj, rope=False)

trigger = None

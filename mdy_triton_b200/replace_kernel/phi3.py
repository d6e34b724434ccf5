"""Patch transformers' Phi3 modules with the fused kernels at import time
(reference: mdy_triton/replace_kernel/phi3.py).  Phi3 projects gate and up with one matrix, so its MLP
uses the no-split SwiGLU; the layer's residual dropouts are kept."""
import importlib

from ._common import mlp_forward_fused_proj, patch_family

module = importlib.import_module("transformers.models.phi3.modeling_phi3")
patch_family(module, "Phi3", mlp=mlp_forward_fused_proj)

trigger = None

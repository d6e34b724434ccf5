"""Patch transformers' Qwen2 modules with the fused kernels at import time
(reference: mdy_triton/replace_kernel/qwen2.py)."""
import importlib

from ._common import patch_family

module = importlib.import_module("transformers.models.qwen2.modeling_qwen2")
patch_family(module, "Qwen2")

trigger = None

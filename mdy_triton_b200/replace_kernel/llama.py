"""Patch transformers' Llama modules with the fused kernels at import time
(reference: mdy_triton/replace_kernel/llama.py)."""
import importlib

from ._common import patch_family

module = importlib.import_module("transformers.models.llama.modeling_llama")
patch_family(module, "Llama")

trigger = None

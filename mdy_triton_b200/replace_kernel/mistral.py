"""Patch transformers' Mistral modules with the fused kernels at import time
(reference: mdy_triton/replace_kernel/mistral.py)."""
import importlib

from ._common import patch_family

module = importlib.import_module("transformers.models.mistral.modeling_mistral")
patch_family(module, "Mistral", fuse_add_norm=False)

trigger = None

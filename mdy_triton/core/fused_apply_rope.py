"""Alias of ``mdy_triton_b200.core.fused_apply_rope`` under the reference's import path."""
import importlib as _importlib

_impl = _importlib.import_module("mdy_triton_b200.core.fused_apply_rope")
globals().update({k: v for k, v in vars(_impl).items() if not k.startswith("__")})

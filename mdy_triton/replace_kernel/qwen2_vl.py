"""Alias of ``mdy_triton_b200.replace_kernel.qwen2_vl`` under the reference's import path."""
from mdy_triton_b200.replace_kernel.qwen2_vl import module, trigger  # noqa: F401

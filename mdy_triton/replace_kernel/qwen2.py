"""Alias of ``mdy_triton_b200.replace_kernel.qwen2`` under the reference's import path."""
from mdy_triton_b200.replace_kernel.qwen2 import module, trigger  # noqa: F401

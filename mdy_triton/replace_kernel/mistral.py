"""Alias of ``mdy_triton_b200.replace_kernel.mistral`` under the reference's import path."""
from mdy_triton_b200.replace_kernel.mistral import module, trigger  # noqa: F401

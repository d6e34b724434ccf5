"""Alias of ``mdy_triton_b200.replace_kernel.llama`` under the reference's import path."""
from mdy_triton_b200.replace_kernel.llama import module, trigger  # noqa: F401

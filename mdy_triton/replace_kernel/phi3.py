"""Alias of ``mdy_triton_b200.replace_kernel.phi3`` under the reference's import path."""
from mdy_triton_b200.replace_kernel.phi3 import module, trigger  # noqa: F401

"""Alias of ``mdy_triton_b200.replace_kernel.glm4`` under the reference's import path."""
from mdy_triton_b200.replace_kernel.glm4 import module, trigger  # noqa: F401

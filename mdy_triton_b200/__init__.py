"""B200-native implementation of the ``mdy_triton.replace_kernel`` hot path.

``mdy_triton_b200.core``            fused operators (same names and signatures as ``mdy_triton.core``)
``mdy_triton_b200.replace_kernel``  import-time patches of HuggingFace Llama/Qwen2/... modules
``mdy_triton_b200._C``              ctypes binding of the C-ABI CUDA library (``include/mdy_kernels.h``)

The top-level package ``mdy_triton`` in this repository re-exports these under the reference's import
paths, so ``from mdy_triton.replace_kernel import *`` keeps working unchanged.
"""
__version__ = "0.1.0"

"""Import-path compatibility package: ``mdy_triton.core`` and ``mdy_triton.replace_kernel`` resolve to
the B200-native implementation in ``mdy_triton_b200`` so that code written against the reference
(``from mdy_triton.replace_kernel import *``, ``from mdy_triton.core import triton_rmsnorm``) runs
unchanged."""

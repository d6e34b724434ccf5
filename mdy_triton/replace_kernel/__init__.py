from mdy_triton_b200.replace_kernel import *  # noqa: F401,F403
from mdy_triton_b200.replace_kernel import trigger, set_residual_fusion, residual_fusion_enabled  # noqa: F401

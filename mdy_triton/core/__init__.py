from mdy_triton_b200.core import *  # noqa: F401,F403
from mdy_triton_b200.core import __all__  # noqa: F401

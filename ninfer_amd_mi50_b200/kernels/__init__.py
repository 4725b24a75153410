"""CUDA kernels for sm_100a and their Python faces.

`from ninfer_amd_mi50_b200 import kernels; kernels.linear(...)`.  Importing this package does not
build or load anything; the first kernel call does.
"""

from .lib import KernelError, is_loaded, load
from .ops import *  # noqa: F401,F403
from .ops import MoePlan, PackedWeights, TUNING, check_attention_limits, check_head_dim, check_router_sizes, check_status, index_status, tensor_core_status

"""Import-compatibility name for :mod:`stacr_b200.fused_kernels` (the kernels are CUDA for sm_100a; Triton is not used)."""

from .fused_kernels import *  # noqa: F401,F403
from .fused_kernels import (kernels_available, projection_pytorch, projection_triton, stacr_forward_fused, stacr_forward_pytorch,  # noqa: F401
                            triton_available, triton_matmul, verify_fused_kernel)

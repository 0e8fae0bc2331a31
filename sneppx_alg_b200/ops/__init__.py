"""Front-ends of the sm_100a kernel library (one autograd function + one PyTorch oracle per op)."""
from . import functional  # noqa: F401
from .functional import *  # noqa: F401,F403
from .gemm import gemm, gemm_reference, linear  # noqa: F401
from ._lib import KernelTimeout, check_status  # noqa: F401

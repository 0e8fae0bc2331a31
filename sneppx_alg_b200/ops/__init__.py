"""Front-ends of the sm_100a kernel library (one autograd function + one PyTorch oracle per op)."""
from . import functional  # noqa: F401
from .functional import *  # noqa: F401,F403
from .gemm import gemm, gemm_reference, linear  # noqa: F401
from ._lib import KernelTimeout, check_status  # noqa: F401
from . import aux  # noqa: F401
from .aux import arc_step, block_top2, dequant_int8, dropout, quant_int8, rng_fill, weighted_average  # noqa: F401

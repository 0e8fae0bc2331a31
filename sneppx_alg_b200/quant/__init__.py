"""Quantisation: algorithms (int8 / int4 / fp8 / AWQ / GPTQ / MX / NVFP4) and the serving kernels' Python API."""
from .algorithms import *  # noqa: F401,F403
from .algorithms import QuantMode  # noqa: F401
from ..ops.quant import (QuantizedLinear, dequant_fp8, dequant_int4, gemm_dequant, quant_fp8_128x128,  # noqa: F401
                         quant_fp8_1x128, quant_int4, quantize_model_)

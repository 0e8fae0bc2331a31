"""Stand-alone ONNX toolkit: protobuf codec, checker, executor, optimiser and exporters (``toolkit``), and the wider
operator set, graph passes, strict checker and convolutional exporter (``ops_ext``, which registers its operators on
import)."""
from .toolkit import *  # noqa: F401,F403
from .ops_ext import (check_model_strict, eliminate_common_subexpressions, eliminate_identity, export_sequential,  # noqa: F401
                      fold_batchnorm_into_conv, fuse_matmul_add, fuse_transposes, run_passes, topological_sort)

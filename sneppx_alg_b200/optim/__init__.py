"""Optimizers: fused AdamW / gradient-norm kernels front-ends and the optimizer zoo."""
from .fused import FusedAdamW, adamw_flat_, adamw_reference, clip_grad_norm_, grad_norm_  # noqa: F401
from .zoo import (SGD, Adam, AdamW, Adamax, RMSprop, Adagrad, Adadelta, RAdam, ScheduleFreeAdamW, Lion, LAMB, LARS,  # noqa: F401
                  AdaFactor, get_optimizer)

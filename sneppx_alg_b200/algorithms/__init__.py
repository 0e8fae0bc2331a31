"""The reference's five pipeline algorithms (HSS, SER, ARC, NPE, FM) and the unified model that chains them."""
from .hss import HSSConfig, HSSDiscretize, HSSModel, HSSScan, HSSStep, DenseHSSLayer  # noqa: F401
from .ser import SERConfig, SERLayer, SERLoss, SERModel, SERRoute  # noqa: F401
from .arc import ARCConfig, ARCLayer, ARCModel, GradientObfuscator, InputGuard, OutputVerifier, simulate_attack  # noqa: F401
from .npe import (NPEConfig, NPELayer, NPEModel, NPEProgram, NPEVM, Instruction, Op, compile_attention,  # noqa: F401
                  compile_mlp, jit_optimize, verify_program)
from .fm import FMConfig, FMController, FMModel, FMSyncNCCL, MemoryBank, compress_topk  # noqa: F401
from .pipeline import Model, ModelConfig, SNEPPXModel  # noqa: F401

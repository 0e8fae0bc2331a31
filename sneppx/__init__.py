"""``import sneppx`` — the package name the reference's documentation uses (``sneppx.nn``, ``sneppx.serving``,
``sneppx.hub``, ``sneppx.distributed``).  Every submodule is the corresponding module of ``sneppx_alg_b200``."""
import importlib
import sys

import sneppx_alg_b200 as _impl
from sneppx_alg_b200 import *  # noqa: F401,F403

_SUB = {"nn": "nn", "ops": "ops", "optim": "optim", "serving": "serving", "hub": "hub", "models": "models",
        "training": "training", "checkpoint": "checkpoint", "quant": "quant", "security": "security", "onnx": "onnx",
        "algorithms": "algorithms", "utils": "utils", "parallel": "parallel", "distributed": "parallel.distributed",
        "cli": "cli", "benchmarks": "benchmarks"}


def __getattr__(name):
    if name in _SUB:
        mod = importlib.import_module(f"sneppx_alg_b200.{_SUB[name]}")
        sys.modules[f"sneppx.{name}"] = mod
        return mod
    return getattr(_impl, name)


__version__ = getattr(_impl, "__version__", "0.1.0")

"""sneppx_alg_b200: a Blackwell (sm_100a) native deep-learning framework with the capabilities of SNEPPX-Alg.

Sub-packages: ``nn`` (layers), ``ops`` (kernel front-ends), ``models`` (model families and presets),
``parallel`` (ZeRO / TP / PP / EP, symmetric memory, elastic runtime), ``optim``, ``training``,
``checkpoint``, ``serving``, ``hub``, ``onnx``, ``quant``, ``security``, ``utils``.
"""
__version__ = "0.1.0"

from . import nn, ops, models  # noqa: F401

"""Compatibility shim for code written against the reference's ``SneppX_ALG`` package: the flat namespace of
``SneppX_ALG.interface_bindings`` re-exported from ``sneppx_alg_b200``."""
from . import interface_bindings as _ib


def __getattr__(name):
    return getattr(_ib, name)

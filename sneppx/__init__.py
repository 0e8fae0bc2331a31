"""``import sneppx`` — the package name the reference's documentation uses (``sneppx.nn``, ``sneppx.serving``,
``sneppx.hub``, ``sneppx.distributed``).  Every submodule is the corresponding module of ``sneppx_alg_b200``:
``sneppx.nn is sneppx_alg_b200.nn``, and ``from sneppx.models.llama import LlamaForCausalLM`` imports
``sneppx_alg_b200.models.llama`` (an import hook maps the names; nothing is copied)."""
import importlib
import importlib.abc
import importlib.util
import sys

import sneppx_alg_b200 as _impl
from sneppx_alg_b200 import *  # noqa: F401,F403

_SUB = {"nn": "nn", "ops": "ops", "optim": "optim", "serving": "serving", "hub": "hub", "models": "models",
        "training": "training", "checkpoint": "checkpoint", "quant": "quant", "security": "security", "onnx": "onnx",
        "algorithms": "algorithms", "utils": "utils", "parallel": "parallel", "distributed": "parallel.distributed",
        "cli": "cli", "benchmarks": "benchmarks"}


def _target(fullname: str):
    parts = fullname.split(".")
    if len(parts) < 2 or parts[0] != __name__:
        return None
    return ".".join(["sneppx_alg_b200", _SUB.get(parts[1], parts[1])] + parts[2:])     # other modules keep their name


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target):
        self.target = target

    def create_module(self, spec):
        mod = importlib.import_module(self.target)           # the real module object, under a second name
        self._keep = {k: getattr(mod, k, None) for k in ("__spec__", "__loader__", "__package__", "__path__", "__file__", "__cached__")}
        return mod

    def exec_module(self, module):
        for k, v in self._keep.items():                      # the import system re-labelled the module: undo that
            if v is not None:
                setattr(module, k, v)


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        real = _target(fullname)
        try:
            if real is None or importlib.util.find_spec(real) is None:
                return None
        except ModuleNotFoundError:                           # a parent package of the target does not exist
            return None
        return importlib.util.spec_from_loader(fullname, _AliasLoader(real))


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())


def __getattr__(name):
    if name in _SUB:
        return importlib.import_module(f"{__name__}.{name}")
    try:
        return getattr(_impl, name)
    except AttributeError:
        if not name.startswith("_"):
            try:
                return importlib.import_module(f"{__name__}.{name}")
            except ModuleNotFoundError:
                pass
        raise


__version__ = getattr(_impl, "__version__", "0.1.0")

"""Shared by the examples: makes the repository importable when the package is not installed, picks the device and
seeds the generators."""
import os
import sys

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if _ROOT not in sys.path:
    sys.path.insert(0, _ROOT)

import torch  # noqa: E402


def device() -> torch.device:
    return torch.device("cuda" if torch.cuda.is_available() else "cpu")


def seed(n: int = 0) -> torch.Generator:
    torch.manual_seed(n)
    return torch.Generator().manual_seed(n)

"""Stand-alone ONNX toolkit."""
from .toolkit import *  # noqa: F401,F403

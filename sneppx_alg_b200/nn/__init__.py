"""``sneppx.nn`` layer vocabulary."""
from .modules import *  # noqa: F401,F403
from .modules import (Module, Linear, Embedding, Dropout, LayerNorm, RMSNorm, GELU, SiLU, ReLU, Sigmoid, Tanh,  # noqa: F401
                      Sequential, MultiheadAttention, TransformerBlock, Transformer, SwiGLU)

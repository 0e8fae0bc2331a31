"""``sneppx.nn``: the layer vocabulary of the reference's Python API
(bindings/python/SneppX_ALG/interface_bindings/nn.py:33-404) on top of ``torch.nn.Module``.

Class names, constructor arguments and defaults follow the reference (``RMSNorm`` eps 1e-6,
pre-LN ``TransformerBlock`` with a GELU FFN, learned positions in ``Transformer``); the forward
passes call the sm_100a kernels for CUDA bf16 tensors and plain PyTorch otherwise.
"""
from __future__ import annotations

import math

import torch
import torch.nn as tnn
import torch.nn.functional as F

from ..ops import functional as ops


class Module(tnn.Module):
    """Base class. Adds the reference's conveniences on top of ``torch.nn.Module``."""

    def num_parameters(self, trainable_only: bool = False) -> int:
        return sum(p.numel() for p in self.parameters() if p.requires_grad or not trainable_only)

    def cuda_bf16(self, device=None):
        return self.to(device=device or "cuda", dtype=torch.bfloat16)


class Linear(Module):
    def __init__(self, in_features, out_features, bias=True, dtype=None, device=None, init_std=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = tnn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device))
        self.bias = tnn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) if bias else None
        if init_std is None:
            tnn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        else:
            tnn.init.normal_(self.weight, std=init_std)

    def forward(self, x):
        return ops.linear(x, self.weight, self.bias)

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"


class Embedding(Module):
    def __init__(self, num_embeddings, embedding_dim, dtype=None, device=None, init_std=0.02):
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.weight = tnn.Parameter(torch.empty(num_embeddings, embedding_dim, dtype=dtype, device=device))
        tnn.init.normal_(self.weight, std=init_std)

    def forward(self, indices):
        return F.embedding(indices, self.weight)


class Dropout(tnn.Dropout, Module):
    """Inverted dropout. On bf16 CUDA activations the keep-mask is a function of (seed, stream offset, element index)
    that backward recomputes, so no mask tensor is stored between the passes (``ops.aux.dropout``). The stream offset
    of a call is drawn from PyTorch's CPU generator: ``torch.manual_seed`` makes runs repeatable, and activation
    checkpointing, which restores that generator before it re-runs a forward, gets the same mask again."""

    def __init__(self, p=0.5, inplace=False, seed=0):
        super().__init__(p, inplace)
        self.seed = seed

    def forward(self, x):
        if self.training and self.p > 0 and x.is_cuda and x.dtype == torch.bfloat16 and x.numel() % 8 == 0:
            from ..ops import aux
            offset = int(torch.randint(0, 2 ** 31 - 1, (1,)).item())
            return aux.dropout(x, self.p, self.seed, offset)
        return super().forward(x)


class LayerNorm(Module):
    def __init__(self, normalized_shape, eps=1e-5, elementwise_affine=True, dtype=None, device=None):
        super().__init__()
        dim = normalized_shape if isinstance(normalized_shape, int) else normalized_shape[-1]
        self.eps = eps
        self.weight = tnn.Parameter(torch.ones(dim, dtype=dtype, device=device))
        self.bias = tnn.Parameter(torch.zeros(dim, dtype=dtype, device=device))
        if not elementwise_affine:
            self.weight.requires_grad_(False)
            self.bias.requires_grad_(False)

    def forward(self, x):
        return ops.layernorm(x, self.weight, self.bias, self.eps)


class RMSNorm(Module):
    def __init__(self, dim, eps=1e-6, dtype=None, device=None):
        super().__init__()
        self.eps = eps
        self.weight = tnn.Parameter(torch.ones(dim, dtype=dtype, device=device))

    def forward(self, x, residual=None):
        y, h = ops.rmsnorm(x, self.weight, self.eps, residual)
        return y if residual is None else (y, h)


class GELU(Module):
    def forward(self, x):
        return F.gelu(x, approximate="tanh")


class SiLU(Module):
    def forward(self, x):
        return F.silu(x)


class ReLU(Module):
    def forward(self, x):
        return F.relu(x)


class Sigmoid(Module):
    def forward(self, x):
        return torch.sigmoid(x)


class Tanh(Module):
    def forward(self, x):
        return torch.tanh(x)


class Sequential(tnn.Sequential, Module):
    pass


class MultiheadAttention(Module):
    """Self-attention with fused QKV projection; ``num_kv_heads`` < ``num_heads`` gives GQA."""

    def __init__(self, embed_dim, num_heads, num_kv_heads=None, bias=False, causal=True, dropout=0.0, dtype=None,
                 device=None, window=0):
        super().__init__()
        self.embed_dim, self.num_heads = embed_dim, num_heads
        self.num_kv_heads = num_kv_heads or num_heads
        self.head_dim = embed_dim // num_heads
        self.causal, self.window = causal, window
        qkv = (self.num_heads + 2 * self.num_kv_heads) * self.head_dim
        self.qkv_proj = Linear(embed_dim, qkv, bias=bias, dtype=dtype, device=device, init_std=0.02)
        self.out_proj = Linear(embed_dim, embed_dim, bias=bias, dtype=dtype, device=device, init_std=0.02)

    def forward(self, x, rope=None, positions=None):
        B, S, _ = x.shape
        H, Hk, D = self.num_heads, self.num_kv_heads, self.head_dim
        qkv = self.qkv_proj(x)
        if rope is not None:
            qkv = ops.rope_qk_(qkv, rope[0], rope[1], H + Hk, D, positions)
        q = qkv[..., : H * D].view(B, S, H, D)
        k = qkv[..., H * D: (H + Hk) * D].view(B, S, Hk, D)
        v = qkv[..., (H + Hk) * D:].view(B, S, Hk, D)
        o = ops.attention(q, k, v, causal=self.causal, window=self.window)
        return self.out_proj(o.reshape(B, S, H * D))


class TransformerBlock(Module):
    """Pre-LN block: x + MHA(LN(x)); x + FFN(LN(x)) with a GELU FFN (nn.py:346-369 of the reference)."""

    def __init__(self, d_model, num_heads, d_ff=None, dropout=0.0, causal=True, dtype=None, device=None):
        super().__init__()
        d_ff = d_ff or 4 * d_model
        self.ln1 = LayerNorm(d_model, dtype=dtype, device=device)
        self.attn = MultiheadAttention(d_model, num_heads, causal=causal, dtype=dtype, device=device)
        self.ln2 = LayerNorm(d_model, dtype=dtype, device=device)
        self.ff1 = Linear(d_model, d_ff, dtype=dtype, device=device)
        self.ff2 = Linear(d_ff, d_model, dtype=dtype, device=device)
        self.drop = Dropout(dropout)

    def forward(self, x):
        x = x + self.drop(self.attn(self.ln1(x)))
        return x + self.drop(self.ff2(F.gelu(self.ff1(self.ln2(x)), approximate="tanh")))


class Transformer(Module):
    """Token + learned position embeddings, N blocks, final LN, untied LM head (nn.py:372-404)."""

    def __init__(self, vocab_size, d_model, num_heads, num_layers, d_ff=None, max_seq_len=512, dropout=0.0,
                 dtype=None, device=None):
        super().__init__()
        self.tok_emb = Embedding(vocab_size, d_model, dtype=dtype, device=device)
        self.pos_emb = Embedding(max_seq_len, d_model, dtype=dtype, device=device)
        self.blocks = tnn.ModuleList(
            [TransformerBlock(d_model, num_heads, d_ff, dropout, dtype=dtype, device=device) for _ in range(num_layers)])
        self.ln_f = LayerNorm(d_model, dtype=dtype, device=device)
        self.head = Linear(d_model, vocab_size, bias=False, dtype=dtype, device=device, init_std=0.02)

    def forward(self, tokens):
        B, S = tokens.shape
        pos = torch.arange(S, device=tokens.device)
        x = self.tok_emb(tokens) + self.pos_emb(pos)[None]
        for blk in self.blocks:
            x = blk(x)
        return self.head(self.ln_f(x))


class SwiGLU(Module):
    """Gated FFN: down(act(gate(x)) * up(x)); gate and up are one fused GEMM. ``act`` in
    {silu, gelu, relu} gives SwiGLU / GeGLU / ReGLU (kernel/activations/gated_activations.c:33-118)."""

    def __init__(self, d_model, d_ff, act="silu", dtype=None, device=None, init_std=0.02):
        super().__init__()
        self.act = act
        self.gate_up_proj = Linear(d_model, 2 * d_ff, bias=False, dtype=dtype, device=device, init_std=init_std)
        self.down_proj = Linear(d_ff, d_model, bias=False, dtype=dtype, device=device, init_std=init_std)

    def forward(self, x):
        return self.down_proj(ops.glu(self.gate_up_proj(x), self.act))

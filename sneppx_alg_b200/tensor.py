"""Tensor / autograd surface of the reference's Python API (``tensor.py``: ``Tensor`` with ``.backward()``, ``.cuda()``,
losses, conv, norms; ``autograd.py``: ``Function`` / ``Context``; ``autograd_ops.py``).  The tensor type IS
``torch.Tensor`` — one device layer, no second array type — and the names below are the reference's spellings."""
from __future__ import annotations

import torch
import torch.nn.functional as F

Tensor = torch.Tensor
Function = torch.autograd.Function
Context = torch.autograd.function.FunctionCtx
no_grad = torch.no_grad
enable_grad = torch.enable_grad


def tensor(data, dtype=None, device=None, requires_grad=False):
    return torch.tensor(data, dtype=dtype, device=device, requires_grad=requires_grad)


zeros, ones, empty, full, arange, randn, rand, eye, linspace = (torch.zeros, torch.ones, torch.empty, torch.full,
                                                                torch.arange, torch.randn, torch.rand, torch.eye,
                                                                torch.linspace)
matmul, cat, stack, where, einsum = torch.matmul, torch.cat, torch.stack, torch.where, torch.einsum
inverse, det = torch.linalg.inv, torch.linalg.det
softmax, log_softmax, relu, gelu, silu, sigmoid, tanh = (torch.softmax, torch.log_softmax, torch.relu, F.gelu, F.silu,
                                                         torch.sigmoid, torch.tanh)
conv1d, conv2d, max_pool2d, avg_pool2d = F.conv1d, F.conv2d, F.max_pool2d, F.avg_pool2d
layer_norm, batch_norm, embedding, dropout = F.layer_norm, F.batch_norm, F.embedding, F.dropout
mse_loss, cross_entropy, binary_cross_entropy, l1_loss = F.mse_loss, F.cross_entropy, F.binary_cross_entropy, F.l1_loss


def fake_quant(x, bits=8):
    """Straight-through fake quantisation (the reference's differentiable ``fake_quant`` op, autodiff/ops.c)."""
    qmax = 2 ** (bits - 1) - 1
    s = x.detach().abs().max().clamp_min(1e-12) / qmax
    q = torch.round(x / s).clamp(-qmax - 1, qmax) * s
    return x + (q - x).detach()


def clip_grad_norm(parameters, max_norm):
    """Global-norm clipping (``SNEPPX_tape_clip_grad_norm``, kernel/autodiff/tape.c:261); one fused reduction on CUDA."""
    from .optim.fused import clip_grad_norm_
    return clip_grad_norm_(parameters, max_norm)


def save(obj, path):
    torch.save(obj, path)


def load(path, map_location="cpu"):
    return torch.load(path, map_location=map_location, weights_only=False)

"""conv2d with a native backward pass (``csrc/conv2d_bwd.cu``).

The forward convolution is PyTorch's (cuDNN on a GPU). The backward pass runs this repository's kernels on CUDA tensors
and, on CPU tensors, the host library's restatement of the same index arithmetic: both include
``csrc/conv2d_bwd_body.h``, so the CPU tests exercise the arithmetic the GPU executes. Square stride and padding,
dilation 1, groups 1. Reference: ``kernel/cuda/autodiff_cuda.cu:620-740``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib
from ._lib import c_int, ptr, stream


def conv2d_backward_reference(x, w, dy, stride: int = 1, padding: int = 0):
    """(dx, dw, db) in fp32 through autograd on fp32 copies: the oracle."""
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    b = torch.zeros(w.shape[0], dtype=torch.float32, device=x.device, requires_grad=True)
    with torch.backends.cudnn.flags(allow_tf32=False):              # a true fp32 oracle: cuDNN defaults to TF32 on GPUs
        F.conv2d(xf, wf, b, stride=stride, padding=padding).backward(dy.float())
    return xf.grad, wf.grad, b.grad


def conv2d_backward(x: torch.Tensor, w: torch.Tensor, dy: torch.Tensor, stride: int = 1, padding: int = 0,
                    need: Tuple[bool, bool, bool] = (True, True, True)):
    """fp32 (dx, dw, db) of ``conv2d(x, w, b, stride, padding)`` for the upstream gradient `dy`; entries of `need`
    that are False come back as None. x [N,C,H,W], w [K,C,R,S], dy [N,K,OH,OW]; fp32 or bf16 (all three alike)."""
    N, Cc, H, W = x.shape
    K, C2, R, S = w.shape
    OH, OW = (H + 2 * padding - R) // stride + 1, (W + 2 * padding - S) // stride + 1
    if C2 != Cc or tuple(dy.shape) != (N, K, OH, OW):
        raise ValueError(f"shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, dy {tuple(dy.shape)}, expected dy {(N, K, OH, OW)}")
    if not (x.device == w.device == dy.device):
        raise ValueError("x, w and dy must live on one device")
    if not (x.dtype == w.dtype == dy.dtype) or x.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError("x, w and dy must share one dtype, fp32 or bf16")
    x, w, dy = x.contiguous(), w.contiguous(), dy.contiguous()
    dev = x.device
    dx = torch.empty(x.shape, dtype=torch.float32, device=dev) if need[0] else None
    dw = torch.empty(w.shape, dtype=torch.float32, device=dev) if need[1] else None
    db = torch.empty(K, dtype=torch.float32, device=dev) if need[2] else None
    dims = [c_int(v) for v in (N, Cc, H, W, K, R, S, stride, padding)]
    if x.is_cuda:
        _lib.call("sx_conv2d_bwd", ptr(x), ptr(w), ptr(dy), ptr(dx), ptr(dw), ptr(db), *dims, c_int(int(x.dtype == torch.bfloat16)), stream())
    else:
        from .. import _build
        L = _build.load_host()
        L.sx_oracle_conv2d_bwd.argtypes = [C.c_void_p] * 6 + [C.c_int] * 9
        xf, wf, dyf = x.float(), w.float(), dy.float()
        rc = L.sx_oracle_conv2d_bwd(ptr(xf), ptr(wf), ptr(dyf), ptr(dx), ptr(dw), ptr(db), *dims)
        if rc != 0:
            raise RuntimeError(f"conv2d backward refused its arguments (code {rc})")
    return dx, dw, db


class _Conv2d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, stride, padding):
        ctx.save_for_backward(x, w)
        ctx.stride, ctx.padding, ctx.has_bias = stride, padding, b is not None
        return F.conv2d(x, w, b, stride=stride, padding=padding)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        need = (ctx.needs_input_grad[0], ctx.needs_input_grad[1], ctx.has_bias and ctx.needs_input_grad[2])
        dx, dw, db = conv2d_backward(x, w, dy.to(x.dtype), ctx.stride, ctx.padding, need)
        cast = lambda g, like: None if g is None else g.to(like.dtype)  # noqa: E731
        return cast(dx, x), cast(dw, w), (None if db is None else db.to(w.dtype)), None, None


def conv2d(x, w, b: Optional[torch.Tensor] = None, stride: int = 1, padding: int = 0):
    """conv2d whose backward pass is this repository's code (see the module docstring for the supported cases)."""
    return _Conv2d.apply(x, w, b, stride, padding)

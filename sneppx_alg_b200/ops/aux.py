"""Front-ends of ``csrc/rng_aux.cu``: counter-based random fills, mask-free dropout, LayerNorm with a native backward,
gradient compression (block int8, block top-2 with error feedback), weighted averaging and adversarial steps.

Each op has a plain PyTorch restatement next to it (``*_reference``) used on CPU tensors and as the test oracle.
Random ops are deterministic functions of ``(seed, offset, element index)`` (Philox4x32-10), so the references
reproduce the device bits by running the same counter arithmetic in integer tensors.

Reference: ``kernel/cuda/rng_cuda.cu``, ``kernel/cuda/autodiff_cuda.cu:331-431``, ``algorithms/fm/cuda/fm_cuda.cu``,
``algorithms/arc/cuda/arc_cuda.cu``.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Sequence

import torch
import torch.nn.functional as F

from . import _lib
from ._lib import c_float, c_int, c_ll, ptr, stream

c_u64 = C.c_ulonglong
_M32 = 0xFFFFFFFF


# ------------------------------------------------------------------------------------------------- Philox oracle
def philox_reference(seed: int, offset: int, nq: int, device="cpu") -> torch.Tensor:
    """[nq, 4] int64 words (values < 2^32): the Philox4x32-10 output for counters (q, offset), key `seed`."""
    q = torch.arange(nq, dtype=torch.int64, device=device)
    c = [q & _M32, q >> 32, torch.full_like(q, offset & _M32), torch.full_like(q, (offset >> 32) & _M32)]
    k0, k1 = seed & _M32, (seed >> 32) & _M32
    M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85

    def mulhilo(m, x):  # 32 x 32 -> (hi, lo) without overflowing int64
        xl, xh = x & 0xFFFF, x >> 16
        ml, mh = m & 0xFFFF, m >> 16
        ll, lh, hl, hh = ml * xl, ml * xh, mh * xl, mh * xh
        mid = (ll >> 16) + (lh & 0xFFFF) + (hl & 0xFFFF)
        lo = ((mid & 0xFFFF) << 16) | (ll & 0xFFFF)
        hi = hh + (lh >> 16) + (hl >> 16) + (mid >> 16)
        return hi & _M32, lo & _M32

    for _ in range(10):
        hi0, lo0 = mulhilo(M0, c[0])
        hi1, lo1 = mulhilo(M1, c[2])
        c = [hi1 ^ c[1] ^ k0, lo1, hi0 ^ c[3] ^ k1, lo0]
        k0, k1 = (k0 + W0) & _M32, (k1 + W1) & _M32
    return torch.stack(c, dim=1)


def _u01(words: torch.Tensor) -> torch.Tensor:
    return ((words >> 8).to(torch.float32) + 0.5) * (1.0 / 16777216.0)


def rng_reference(n: int, mode: str, a: float, b: float, seed: int, offset: int = 0, device="cpu") -> torch.Tensor:
    w = philox_reference(seed, offset, (n + 3) // 4, device)
    u = _u01(w)
    if mode == "uniform":
        out = a + (b - a) * u
    elif mode == "bernoulli":
        out = (u < a).float()
    else:
        r0, r1 = torch.sqrt(-2.0 * torch.log(u[:, 0])), torch.sqrt(-2.0 * torch.log(u[:, 2]))
        t0, t1 = 2 * math.pi * u[:, 1], 2 * math.pi * u[:, 3]
        out = a + b * torch.stack([r0 * torch.cos(t0), r0 * torch.sin(t0), r1 * torch.cos(t1), r1 * torch.sin(t1)], 1)
    return out.reshape(-1)[:n]


_MODES = {"uniform": 0, "normal": 1, "bernoulli": 2}


def rng_fill(n: int, mode: str = "uniform", a: float = 0.0, b: float = 1.0, seed: int = 0, offset: int = 0,
             device="cuda") -> torch.Tensor:
    """fp32 [n]: uniform [a, b), normal(mean a, std b) or bernoulli(p = a)."""
    dev = torch.device(device)
    if dev.type != "cuda" or not _lib.available():
        return rng_reference(n, mode, a, b, seed, offset, dev)
    out = torch.empty(n, dtype=torch.float32, device=dev)
    _lib.call("sx_rng_fill", ptr(out), c_ll(n), c_int(_MODES[mode]), c_float(a), c_float(b), c_u64(seed), c_u64(offset), stream())
    return out


# ------------------------------------------------------------------------------------------------------ dropout
def dropout_mask_reference(n: int, p: float, seed: int, offset: int, device="cpu") -> torch.Tensor:
    return (_u01(philox_reference(seed, offset, (n + 3) // 4, device)).reshape(-1)[:n] >= p)


def dropout_reference(x, p, seed, offset=0):
    keep = dropout_mask_reference(x.numel(), p, seed, offset, x.device).view(x.shape)
    return (x.float() * keep / (1.0 - p)).to(x.dtype)


class _DropoutFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p, seed, offset):
        ctx.p, ctx.seed, ctx.offset = p, seed, offset
        x = x.contiguous()
        y = torch.empty_like(x)
        _lib.call("sx_dropout", ptr(x), ptr(y), c_ll(x.numel()), c_float(p), c_u64(seed), c_u64(offset), stream())
        return y

    @staticmethod
    def backward(ctx, dy):
        dy = dy.contiguous()
        dx = torch.empty_like(dy)
        _lib.call("sx_dropout", ptr(dy), ptr(dx), c_ll(dy.numel()), c_float(ctx.p), c_u64(ctx.seed), c_u64(ctx.offset), stream())
        return dx, None, None, None


def dropout(x, p: float, seed: int, offset: int = 0, training: bool = True):
    """Inverted dropout whose keep-mask is recomputed from (seed, offset) in backward instead of being stored."""
    if not training or p == 0.0:
        return x
    if x.is_cuda and x.dtype == torch.bfloat16 and x.numel() % 8 == 0 and _lib.available():
        return _DropoutFn.apply(x, float(p), int(seed), int(offset))
    keep = dropout_mask_reference(x.numel(), p, seed, offset, x.device).view(x.shape)
    return x * keep.to(x.dtype) / (1.0 - p)


# ---------------------------------------------------------------------------------------------------- LayerNorm
class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps):
        d = x.shape[-1]
        x2 = x.reshape(-1, d).contiguous()
        y = torch.empty_like(x2)
        mean = torch.empty(x2.shape[0], dtype=torch.float32, device=x2.device)
        rstd = torch.empty_like(mean)
        _lib.call("sx_layernorm_fwd", ptr(x2), ptr(w), ptr(b), ptr(y), ptr(mean), ptr(rstd), c_ll(x2.shape[0]), c_int(d),
                  c_float(eps), stream())
        ctx.save_for_backward(x2, w, mean, rstd)
        ctx.eps, ctx.has_bias, ctx.shape = eps, b is not None, x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, mean, rstd = ctx.saved_tensors
        rows, d = x2.shape
        dy2 = dy.reshape(rows, d).contiguous()
        dx = torch.empty_like(x2)
        nblk = _lib.lib().sx_layernorm_bwd_blocks(c_ll(rows))
        partials = torch.empty(nblk, 2, d, dtype=torch.float32, device=x2.device)
        dwb = torch.empty(2, d, dtype=torch.float32, device=x2.device)
        gamma = w.float().contiguous()
        _lib.call("sx_layernorm_bwd", ptr(x2), ptr(dy2), ptr(gamma), ptr(mean), ptr(rstd), ptr(dx), ptr(partials), ptr(dwb),
                  c_ll(rows), c_int(d), stream())
        return dx.view(ctx.shape), dwb[0].to(w.dtype), (dwb[1].to(w.dtype) if ctx.has_bias else None), None


def layernorm_train(x, w, b=None, eps=1e-5):
    """LayerNorm with native forward and backward (bf16 CUDA, last dim a multiple of 8); otherwise PyTorch."""
    d = x.shape[-1]
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and d % 8 == 0 and d <= 8192 and _lib.available():
        return _LayerNormFn.apply(x, w, b, eps)
    return F.layer_norm(x, (d,), w, b, eps)


# ------------------------------------------------------------------------------------------- FM compression
def quant_int8_reference(x):
    xb = x.float().reshape(-1, 256)
    m = xb.abs().amax(1)
    inv = torch.where(m > 0, 127.0 / m, torch.zeros_like(m))
    q = torch.clamp(torch.round(xb * inv[:, None]), -127, 127).to(torch.int8)
    return q.reshape(-1), m / 127.0


def quant_int8(x: torch.Tensor):
    """fp32 [n] (n % 256 == 0) -> (int8 [n], fp32 scales [n / 256])."""
    if not (x.is_cuda and _lib.available()):
        return quant_int8_reference(x)
    x = x.float().contiguous().reshape(-1)
    q = torch.empty(x.numel(), dtype=torch.int8, device=x.device)
    s = torch.empty(x.numel() // 256, dtype=torch.float32, device=x.device)
    _lib.call("sx_fm_quant_int8", ptr(x), ptr(q), ptr(s), c_ll(x.numel()), stream())
    return q, s


def dequant_int8(q: torch.Tensor, scales: torch.Tensor):
    if not (q.is_cuda and _lib.available()):
        return (q.reshape(-1, 256).float() * scales[:, None]).reshape(-1)
    y = torch.empty(q.numel(), dtype=torch.float32, device=q.device)
    _lib.call("sx_fm_dequant_int8", ptr(q.contiguous()), ptr(scales.contiguous()), ptr(y), c_ll(q.numel()), stream())
    return y


def block_top2_reference(x):
    xb = x.float().reshape(-1, 32)
    # stable: among equal magnitudes the lowest index wins
    order = torch.sort(xb.abs(), dim=1, descending=True, stable=True).indices[:, :2]
    keep = torch.zeros_like(xb, dtype=torch.bool).scatter_(1, order, True)
    kept = torch.where(keep, xb, torch.zeros_like(xb))
    return kept.reshape(-1), (xb - kept).reshape(-1)


def block_top2(x: torch.Tensor):
    """fp32 [n] (n % 32 == 0) -> (kept, residual): per 32 values the two largest magnitudes, and what was dropped."""
    if not (x.is_cuda and _lib.available()):
        return block_top2_reference(x)
    x = x.float().contiguous().reshape(-1)
    kept, res = torch.empty_like(x), torch.empty_like(x)
    _lib.call("sx_fm_block_top2", ptr(x), ptr(kept), ptr(res), c_ll(x.numel()), stream())
    return kept, res


def weighted_average(tensors: Sequence[torch.Tensor], weights: Sequence[float]) -> torch.Tensor:
    """sum_i w_i * x_i over up to 16 fp32 buffers in one pass."""
    t0 = tensors[0]
    if not (t0.is_cuda and _lib.available()) or len(tensors) > 16 or t0.numel() % 4:
        return sum(w * t.float() for w, t in zip(weights, tensors))
    ts = [t.float().contiguous() for t in tensors]
    arr = (C.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
    ws = (C.c_float * len(ts))(*[float(w) for w in weights])
    out = torch.empty_like(ts[0])
    _lib.call("sx_fm_weighted_avg", arr, ws, c_int(len(ts)), ptr(out), c_ll(out.numel()), stream())
    return out


# ----------------------------------------------------------------------------------------------- ARC steps
_ARC = {"fgsm": 0, "pgd": 1, "obfuscate": 2, "smooth": 3}


def arc_step_reference(mode, x, g=None, x0=None, eps=0.0, alpha=0.0, lo=0.0, hi=1.0, seed=0, offset=0):
    x = x.float()
    if mode == "fgsm":
        return torch.clamp(x + eps * torch.sign(g.float()), lo, hi)
    if mode == "pgd":
        t = x + alpha * torch.sign(g.float())
        return torch.clamp(torch.minimum(torch.maximum(t, x0.float() - eps), x0.float() + eps), lo, hi)
    if mode == "obfuscate":
        return x + eps * torch.sin(100.0 * x)
    z = rng_reference(x.numel(), "normal", 0.0, 1.0, seed, offset, x.device).view(x.shape)
    return x + eps * z


def arc_step(mode: str, x, g: Optional[torch.Tensor] = None, x0: Optional[torch.Tensor] = None, eps=0.0, alpha=0.0,
             lo=0.0, hi=1.0, seed=0, offset=0):
    """One elementwise adversarial step; see ``arc_step_reference`` for the formulas."""
    if not (x.is_cuda and x.numel() % 4 == 0 and _lib.available()):
        return arc_step_reference(mode, x, g, x0, eps, alpha, lo, hi, seed, offset)
    xs = x.float().contiguous()
    out = torch.empty_like(xs)
    gg = None if g is None else g.float().contiguous()
    cc = None if x0 is None else x0.float().contiguous()
    _lib.call("sx_arc_step", ptr(xs), ptr(gg), ptr(cc), ptr(out), c_ll(xs.numel()), c_int(_ARC[mode]), c_float(eps),
              c_float(alpha), c_float(lo), c_float(hi), c_u64(seed), c_u64(offset), stream())
    return out

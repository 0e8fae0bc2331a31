"""O1/O2 front-ends: fused AdamW over flat buffers or tensor lists, gradient-norm clipping.

Update rule and order follow the reference (interface_bindings/optim.py:96-114,
kernel/cuda/optim_cuda.cu:167-207): moments, bias correction, ``p -= lr*wd*p``, then
``p -= lr*m_hat/(sqrt(v_hat)+eps)``. Master weights and moments are fp32; the bf16 copy the model
computes with is written by the same kernel.
"""
from __future__ import annotations

import ctypes as C

import torch

from ..ops import _lib
from ..ops._lib import c_float, c_int, c_ll, ptr, stream


def adamw_reference(p, m, v, g, lr, beta1, beta2, eps, wd, step, grad_scale=1.0):
    """In-place fp32 AdamW on tensors (CPU path and test oracle)."""
    g = g.float() * grad_scale
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    mh = m / (1 - beta1 ** step)
    vh = v / (1 - beta2 ** step)
    p.mul_(1 - lr * wd)
    p.sub_(lr * mh / (vh.sqrt() + eps))
    return p


def adamw_flat_(p32, m, v, g, p16, lr, beta1, beta2, eps, wd, step, grad_scale=1.0, clip=None):
    """One launch for a whole flat shard. ``clip``: optional device scalar multiplying the gradient."""
    if p32.is_cuda and _lib.available():
        _lib.call("sx_adamw_flat", ptr(p32), ptr(m), ptr(v), ptr(g), c_int(int(g.dtype == torch.bfloat16)), ptr(p16),
                  c_ll(p32.numel()), c_float(lr), c_float(beta1), c_float(beta2), c_float(eps), c_float(wd),
                  c_int(step), c_float(grad_scale), ptr(clip), stream())
        return
    gs = grad_scale * (float(clip) if clip is not None else 1.0)
    adamw_reference(p32, m, v, g, lr, beta1, beta2, eps, wd, step, gs)
    if p16 is not None:
        p16.copy_(p32)


_scratch = {}


def _norm_scratch(device):
    key = str(device)
    if key not in _scratch:
        _scratch[key] = (torch.empty(1024, dtype=torch.float32, device=device),
                         torch.zeros(4, dtype=torch.float32, device=device),
                         torch.zeros(1, dtype=torch.int32, device=device))
    return _scratch[key]


def grad_norm_(grads, max_norm=0.0):
    """L2 norm over a list of gradient tensors without a host sync.

    Returns ``out`` (device float32[3]: sum of squares, norm, clip coefficient) and the non-finite flag
    tensor. The clip coefficient is min(1, max_norm/(norm+1e-6)) when ``max_norm`` > 0, else 1.
    """
    grads = [g for g in grads if g is not None and g.numel()]
    dev = grads[0].device
    if dev.type == "cuda" and _lib.available():
        partials, out, flag = _norm_scratch(dev)
        flag.zero_()
        for i, g in enumerate(grads):
            g = g if g.is_contiguous() else g.contiguous()
            last = i == len(grads) - 1
            _lib.call("sx_grad_sumsq", ptr(g), c_int(int(g.dtype == torch.bfloat16)), c_ll(g.numel()), ptr(partials),
                      ptr(out), ptr(flag), c_int(int(i > 0)), c_int(int(last)), c_float(max_norm), stream())
        return out, flag
    ss = sum(float(g.float().pow(2).sum()) for g in grads)
    nrm = ss ** 0.5
    coef = max_norm / (nrm + 1e-6) if (max_norm > 0 and nrm > max_norm) else 1.0
    out = torch.tensor([ss, nrm, coef], dtype=torch.float32, device=dev)
    bad = any(not bool(torch.isfinite(g).all()) for g in grads)
    return out, torch.tensor([int(bad)], dtype=torch.int32, device=dev)


def clip_grad_norm_(parameters, max_norm):
    """torch-style helper: scales ``.grad`` in place, returns the total norm (device scalar)."""
    params = [p for p in parameters if p.grad is not None]
    if not params:
        return torch.tensor(0.0)
    out, _ = grad_norm_([p.grad for p in params], max_norm)
    for p in params:
        p.grad.mul_(out[2].to(p.grad.dtype))
    return out[1]


class FusedAdamW(torch.optim.Optimizer):
    """AdamW over arbitrary parameter lists. CUDA parameters are updated by the multi-tensor kernel
    (fp32 master copy + moments kept in the state, bf16 parameter rewritten in the same pass)."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            b1, b2 = group["betas"]
            todo = []
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["master"] = p.detach().float().clone() if p.dtype != torch.float32 else p.data
                    st["m"] = torch.zeros_like(st["master"])
                    st["v"] = torch.zeros_like(st["master"])
                st["step"] += 1
                todo.append((p, st))
            if not todo:
                continue
            step = todo[0][1]["step"]
            cuda = todo[0][0].is_cuda and _lib.available()
            same = all(t[0].grad.dtype == todo[0][0].grad.dtype and t[1]["step"] == step for t in todo)
            if cuda and same:
                n = len(todo)
                P = (C.c_void_p * n)(*[t[1]["master"].data_ptr() for t in todo])
                M = (C.c_void_p * n)(*[t[1]["m"].data_ptr() for t in todo])
                V = (C.c_void_p * n)(*[t[1]["v"].data_ptr() for t in todo])
                G = (C.c_void_p * n)(*[t[0].grad.contiguous().data_ptr() for t in todo])
                P16 = (C.c_void_p * n)(*[(t[0].data_ptr() if t[0].dtype == torch.bfloat16 else 0) for t in todo])
                N = (C.c_longlong * n)(*[t[0].numel() for t in todo])
                WD = (C.c_float * n)(*[group["weight_decay"]] * n)
                _lib.call("sx_adamw_multi", P, M, V, G, c_int(int(todo[0][0].grad.dtype == torch.bfloat16)), P16, N, WD,
                          c_int(n), c_float(group["lr"]), c_float(b1), c_float(b2), c_float(group["eps"]), c_int(step),
                          c_float(1.0), ptr(None), stream())
                for p, st in todo:
                    if p.dtype not in (torch.bfloat16, torch.float32):
                        p.copy_(st["master"])
            else:
                for p, st in todo:
                    adamw_reference(st["master"], st["m"], st["v"], p.grad, group["lr"], b1, b2, group["eps"],
                                    group["weight_decay"], st["step"])
                    if st["master"] is not p.data:
                        p.copy_(st["master"])
        return loss

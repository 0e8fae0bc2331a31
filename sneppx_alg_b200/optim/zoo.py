"""Optimizer zoo with the reference's names: SGD(+momentum/nesterov), Adam, AdamW, Adamax, RMSprop, Adagrad, Adadelta,
RAdam, schedule-free AdamW (kernel/optimizer/*.c), Lion, LAMB, LARS, AdaFactor (kernel/cuda/optim_cuda.cu:61-482,
interface_bindings/optim_extra.py), ``get_optimizer`` (optim_advanced.py). AdamW / SGD / Lion on CUDA run the fused
kernels in ``csrc/optim.cu``; the rest are compact PyTorch implementations (off the hot path of the benchmarks)."""
from __future__ import annotations

import math

import torch
from torch.optim import Optimizer

from ..ops import _lib
from ..ops._lib import c_float, c_int, c_ll, ptr, stream
from .fused import FusedAdamW

AdamW = FusedAdamW


class SGD(Optimizer):
    def __init__(self, params, lr=1e-2, momentum=0.0, weight_decay=0.0, nesterov=False):
        super().__init__(params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay, nesterov=nesterov))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure else None
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if g["momentum"] and "buf" not in st:
                    st["buf"] = torch.zeros_like(p, dtype=torch.float32)
                if p.is_cuda and p.dtype == torch.float32 and p.grad.dtype == torch.float32 and _lib.available():
                    _lib.call("sx_sgd", ptr(p), ptr(st.get("buf")), ptr(p.grad.contiguous()), ptr(None), c_ll(p.numel()),
                              c_float(g["lr"]), c_float(g["momentum"]), c_float(g["weight_decay"]),
                              c_int(int(g["nesterov"])), stream())
                    continue
                d = p.grad.float() + g["weight_decay"] * p.float()
                if g["momentum"]:
                    buf = st["buf"].mul_(g["momentum"]).add_(d)
                    d = d + g["momentum"] * buf if g["nesterov"] else buf
                p.add_((-g["lr"] * d).to(p.dtype))
        return loss


class Lion(Optimizer):
    def __init__(self, params, lr=1e-4, betas=(0.9, 0.99), weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure else None
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if "m" not in st:
                    st["m"] = torch.zeros_like(p, dtype=torch.float32)
                if p.is_cuda and p.dtype == torch.float32 and p.grad.dtype == torch.float32 and _lib.available():
                    _lib.call("sx_lion", ptr(p), ptr(st["m"]), ptr(p.grad.contiguous()), ptr(None), c_ll(p.numel()),
                              c_float(g["lr"]), c_float(b1), c_float(b2), c_float(g["weight_decay"]), stream())
                    continue
                gr = p.grad.float()
                u = (b1 * st["m"] + (1 - b1) * gr).sign()
                p.add_((-g["lr"] * (u + g["weight_decay"] * p.float())).to(p.dtype))
                st["m"].mul_(b2).add_(gr, alpha=1 - b2)
        return loss


class _Simple(Optimizer):
    """Shared scaffolding: subclasses implement ``update(p32, grad32, state, group) -> new p32``."""

    def __init__(self, params, **defaults):
        super().__init__(params, defaults)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure else None
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                st["step"] = st.get("step", 0) + 1
                new = self.update(p.float(), p.grad.float(), st, g)
                p.copy_(new.to(p.dtype))
        return loss


class Adam(_Simple):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)

    def update(self, p, g, st, grp):
        b1, b2 = grp["betas"]
        g = g + grp["weight_decay"] * p
        m = st.setdefault("m", torch.zeros_like(p)).mul_(b1).add_(g, alpha=1 - b1)
        v = st.setdefault("v", torch.zeros_like(p)).mul_(b2).addcmul_(g, g, value=1 - b2)
        t = st["step"]
        return p - grp["lr"] * (m / (1 - b1 ** t)) / ((v / (1 - b2 ** t)).sqrt() + grp["eps"])


class Adamax(_Simple):
    def __init__(self, params, lr=2e-3, betas=(0.9, 0.999), eps=1e-8):
        super().__init__(params, lr=lr, betas=betas, eps=eps)

    def update(self, p, g, st, grp):
        b1, b2 = grp["betas"]
        m = st.setdefault("m", torch.zeros_like(p)).mul_(b1).add_(g, alpha=1 - b1)
        u = st.setdefault("u", torch.zeros_like(p))
        torch.maximum(u * b2, g.abs(), out=u)
        return p - grp["lr"] / (1 - b1 ** st["step"]) * m / (u + grp["eps"])


class RMSprop(_Simple):
    def __init__(self, params, lr=1e-2, alpha=0.99, eps=1e-8):
        super().__init__(params, lr=lr, alpha=alpha, eps=eps)

    def update(self, p, g, st, grp):
        v = st.setdefault("v", torch.zeros_like(p)).mul_(grp["alpha"]).addcmul_(g, g, value=1 - grp["alpha"])
        return p - grp["lr"] * g / (v.sqrt() + grp["eps"])


class Adagrad(_Simple):
    def __init__(self, params, lr=1e-2, eps=1e-10):
        super().__init__(params, lr=lr, eps=eps)

    def update(self, p, g, st, grp):
        v = st.setdefault("v", torch.zeros_like(p)).addcmul_(g, g)
        return p - grp["lr"] * g / (v.sqrt() + grp["eps"])


class Adadelta(_Simple):
    def __init__(self, params, lr=1.0, rho=0.9, eps=1e-6):
        super().__init__(params, lr=lr, rho=rho, eps=eps)

    def update(self, p, g, st, grp):
        rho, eps = grp["rho"], grp["eps"]
        v = st.setdefault("v", torch.zeros_like(p)).mul_(rho).addcmul_(g, g, value=1 - rho)
        d = st.setdefault("d", torch.zeros_like(p))
        upd = (d + eps).sqrt() / (v + eps).sqrt() * g
        d.mul_(rho).addcmul_(upd, upd, value=1 - rho)
        return p - grp["lr"] * upd


class RAdam(_Simple):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)

    def update(self, p, g, st, grp):
        b1, b2 = grp["betas"]
        t = st["step"]
        m = st.setdefault("m", torch.zeros_like(p)).mul_(b1).add_(g, alpha=1 - b1)
        v = st.setdefault("v", torch.zeros_like(p)).mul_(b2).addcmul_(g, g, value=1 - b2)
        mh = m / (1 - b1 ** t)
        rho_inf = 2 / (1 - b2) - 1
        rho_t = rho_inf - 2 * t * b2 ** t / (1 - b2 ** t)
        p = p * (1 - grp["lr"] * grp["weight_decay"])
        if rho_t > 5:
            r = math.sqrt((rho_t - 4) * (rho_t - 2) * rho_inf / ((rho_inf - 4) * (rho_inf - 2) * rho_t))
            return p - grp["lr"] * r * mh / ((v / (1 - b2 ** t)).sqrt() + grp["eps"])
        return p - grp["lr"] * mh


class ScheduleFreeAdamW(_Simple):
    """Schedule-free AdamW (kernel/optimizer/optimizer_sf_adamw.c): iterate y interpolates the averaged x and z."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, warmup_steps=0):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, warmup_steps=warmup_steps)

    def update(self, p, g, st, grp):
        b1, b2 = grp["betas"]
        t = st["step"]
        z = st.setdefault("z", p.clone())
        x = st.setdefault("x", p.clone())
        v = st.setdefault("v", torch.zeros_like(p)).mul_(b2).addcmul_(g, g, value=1 - b2)
        lr = grp["lr"] * min(1.0, t / max(1, grp["warmup_steps"])) * math.sqrt(1 - b2 ** t)
        st["wsum"] = st.get("wsum", 0.0) + lr ** 2
        c = lr ** 2 / st["wsum"]
        z.sub_(lr * (g / (v.sqrt() + grp["eps"]) + grp["weight_decay"] * p))
        x.mul_(1 - c).add_(z, alpha=c)
        return b1 * x + (1 - b1) * z


class LAMB(_Simple):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.01):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)

    def update(self, p, g, st, grp):
        b1, b2 = grp["betas"]
        t = st["step"]
        m = st.setdefault("m", torch.zeros_like(p)).mul_(b1).add_(g, alpha=1 - b1)
        v = st.setdefault("v", torch.zeros_like(p)).mul_(b2).addcmul_(g, g, value=1 - b2)
        upd = (m / (1 - b1 ** t)) / ((v / (1 - b2 ** t)).sqrt() + grp["eps"]) + grp["weight_decay"] * p
        wn, un = p.norm(), upd.norm()
        trust = (wn / un).item() if wn > 0 and un > 0 else 1.0
        return p - grp["lr"] * trust * upd


class LARS(_Simple):
    def __init__(self, params, lr=0.1, momentum=0.9, weight_decay=1e-4, trust_coef=1e-3):
        super().__init__(params, lr=lr, momentum=momentum, weight_decay=weight_decay, trust_coef=trust_coef)

    def update(self, p, g, st, grp):
        wn, gn = p.norm(), g.norm()
        local = grp["trust_coef"] * wn / (gn + grp["weight_decay"] * wn + 1e-12) if wn > 0 and gn > 0 else 1.0
        buf = st.setdefault("buf", torch.zeros_like(p)).mul_(grp["momentum"]).add_(
            (g + grp["weight_decay"] * p) * (grp["lr"] * local))
        return p - buf


class AdaFactor(_Simple):
    def __init__(self, params, lr=1e-3, beta2=0.999, eps=1e-30, clip=1.0, weight_decay=0.0):
        super().__init__(params, lr=lr, beta2=beta2, eps=eps, clip=clip, weight_decay=weight_decay)

    def update(self, p, g, st, grp):
        b2, eps = grp["beta2"], grp["eps"]
        g2 = g * g + eps
        if p.dim() >= 2:
            r = st.setdefault("r", torch.zeros(p.shape[:-1], device=p.device)).mul_(b2).add_(g2.mean(-1), alpha=1 - b2)
            c = st.setdefault("c", torch.zeros(p.shape[:-2] + p.shape[-1:], device=p.device)).mul_(b2).add_(
                g2.mean(-2), alpha=1 - b2)
            v = r.unsqueeze(-1) * c.unsqueeze(-2) / r.mean(-1, keepdim=True).unsqueeze(-1)
        else:
            v = st.setdefault("v", torch.zeros_like(p)).mul_(b2).add_(g2, alpha=1 - b2)
        u = g / v.sqrt()
        u = u / max(1.0, (u.pow(2).mean().sqrt() / grp["clip"]).item())
        return p * (1 - grp["lr"] * grp["weight_decay"]) - grp["lr"] * u


_REGISTRY = {"sgd": SGD, "adam": Adam, "adamw": AdamW, "adamax": Adamax, "rmsprop": RMSprop, "adagrad": Adagrad,
             "adadelta": Adadelta, "radam": RAdam, "sf_adamw": ScheduleFreeAdamW, "schedule_free_adamw": ScheduleFreeAdamW,
             "lion": Lion, "lamb": LAMB, "lars": LARS, "adafactor": AdaFactor}


def get_optimizer(name: str, params, **kw):
    try:
        cls = _REGISTRY[name.lower()]
    except KeyError as e:
        raise ValueError(f"unknown optimizer '{name}'; available: {sorted(_REGISTRY)}") from e
    import inspect
    ok = set(inspect.signature(cls.__init__).parameters)
    if "betas" in kw and isinstance(kw["betas"], list):
        kw["betas"] = tuple(kw["betas"])
    return cls(params, **{k: v for k, v in kw.items() if k in ok})

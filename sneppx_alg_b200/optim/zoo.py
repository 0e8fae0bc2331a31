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



class SM3(_Simple):
    """Memory-efficient adaptive method: one accumulator per row and per column of a matrix (full accumulator for
    vectors); nu = min(row, col) + g^2 (the reference's ``optim_advanced.SM3``)."""

    def __init__(self, params, lr=0.1, momentum=0.0, eps=1e-30, weight_decay=0.0):
        super().__init__(params, lr=lr, momentum=momentum, eps=eps, weight_decay=weight_decay)

    def update(self, p, g, st, grp):
        if p.dim() == 2:
            r = st.setdefault("row", torch.zeros(p.shape[0], 1, device=p.device))
            c = st.setdefault("col", torch.zeros(1, p.shape[1], device=p.device))
            nu = torch.minimum(r, c) + g * g
            st["row"], st["col"] = nu.amax(1, keepdim=True), nu.amax(0, keepdim=True)
        else:
            nu = st.setdefault("acc", torch.zeros_like(p)).add_(g * g)
        u = g / (nu.sqrt() + grp["eps"])
        if grp["momentum"]:
            u = st.setdefault("m", torch.zeros_like(p)).mul_(grp["momentum"]).add_(u, alpha=1 - grp["momentum"])
        return p * (1 - grp["lr"] * grp["weight_decay"]) - grp["lr"] * u


class Demeter(_Simple):
    """Adam whose second moment of a matrix gradient is a rank-r estimate from two power iterations
    (``optim_advanced.Demeter``): v tracks the low-rank reconstruction U diag(S) V^T squared."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, rank=8):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, rank=rank)

    def update(self, p, g, st, grp):
        b1, b2 = grp["betas"]
        t = st["step"]
        m = st.setdefault("m", torch.zeros_like(p)).mul_(b1).add_(g, alpha=1 - b1)
        if p.dim() == 2:
            r = min(grp["rank"], *p.shape)
            V = st.get("V")
            if V is None:
                V = torch.randn(p.shape[1], r, device=p.device, generator=None) * 0.01
            for _ in range(2):
                U = torch.linalg.qr(g @ V).Q
                V = torch.linalg.qr(g.T @ U).Q
            st["V"] = V
            low = U @ (U.T @ g)
            sq = low * low
        else:
            sq = g * g
        v = st.setdefault("v", torch.zeros_like(p)).mul_(b2).add_(sq, alpha=1 - b2)
        u = (m / (1 - b1 ** t)) / ((v / (1 - b2 ** t)).sqrt() + grp["eps"])
        return p * (1 - grp["lr"] * grp["weight_decay"]) - grp["lr"] * u.clamp(-10, 10)


class CaProp(_Simple):
    """Cautious RMS-style update: the step grows by ``cautious_factor`` x max(0, cos(g, m)) when the gradient agrees
    with its running mean (``optim_advanced.CaProp``; one beta for both moments)."""

    def __init__(self, params, lr=1e-3, beta=0.9, eps=1e-8, weight_decay=0.0, cautious_factor=0.5):
        super().__init__(params, lr=lr, beta=beta, eps=eps, weight_decay=weight_decay, cautious_factor=cautious_factor)

    def update(self, p, g, st, grp):
        b, t = grp["beta"], st["step"]
        m = st.setdefault("m", torch.zeros_like(p)).mul_(b).add_(g, alpha=1 - b)
        v = st.setdefault("v", torch.zeros_like(p)).mul_(b).addcmul_(g, g, value=1 - b)
        bc = 1 - b ** t
        mh, vh = m / bc, v / bc
        align = (g * mh).sum() / (g.norm() * mh.norm() + grp["eps"])
        scale = 1.0 + grp["cautious_factor"] * align.clamp_min(0)
        return p - grp["lr"] * (scale * mh / (vh.sqrt() + grp["eps"]) + grp["weight_decay"] * p)


class SOAP(_Simple):
    """Adam run in the eigenbasis of the Shampoo preconditioners L = E[G G^T], R = E[G^T G]; the bases are refreshed
    every ``precondition_frequency`` steps (``optim_advanced.SOAP``)."""

    def __init__(self, params, lr=3e-3, betas=(0.95, 0.95), eps=1e-8, weight_decay=0.01, shampoo_beta=0.95,
                 precondition_frequency=10, max_dim=4096):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, shampoo_beta=shampoo_beta,
                         precondition_frequency=precondition_frequency, max_dim=max_dim)

    def update(self, p, g, st, grp):
        b1, b2 = grp["betas"]
        t = st["step"]
        rot = p.dim() == 2 and max(p.shape) <= grp["max_dim"]
        if rot:
            sb = grp["shampoo_beta"]
            L = st.setdefault("L", torch.zeros(p.shape[0], p.shape[0], device=p.device)).mul_(sb).add_(g @ g.T, alpha=1 - sb)
            R = st.setdefault("R", torch.zeros(p.shape[1], p.shape[1], device=p.device)).mul_(sb).add_(g.T @ g, alpha=1 - sb)
            if "QL" not in st or t % grp["precondition_frequency"] == 0:
                st["QL"], st["QR"] = torch.linalg.eigh(L).eigenvectors, torch.linalg.eigh(R).eigenvectors
            g = st["QL"].T @ g @ st["QR"]
        m = st.setdefault("m", torch.zeros_like(p)).mul_(b1).add_(g, alpha=1 - b1)
        v = st.setdefault("v", torch.zeros_like(p)).mul_(b2).addcmul_(g, g, value=1 - b2)
        u = (m / (1 - b1 ** t)) / ((v / (1 - b2 ** t)).sqrt() + grp["eps"])
        if rot:
            u = st["QL"] @ u @ st["QR"].T
        return p * (1 - grp["lr"] * grp["weight_decay"]) - grp["lr"] * u


class OrthoAdam(_Simple):
    """Adam-normalised step along the gradient component orthogonal to the last ``history_size`` gradients
    (``optim_advanced.OrthoAdam``)."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, history_size=3):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, history_size=history_size)

    def update(self, p, g, st, grp):
        b1, b2 = grp["betas"]
        t = st["step"]
        st.setdefault("m", torch.zeros_like(p)).mul_(b1).add_(g, alpha=1 - b1)
        v = st.setdefault("v", torch.zeros_like(p)).mul_(b2).addcmul_(g, g, value=1 - b2)
        hist = st.setdefault("hist", [])
        og, basis = g.clone(), []
        for h in hist:                                   # Gram-Schmidt over the history, then project it out
            u = h.clone()
            for q in basis:
                u -= (u * q).sum() / ((q * q).sum() + 1e-12) * q
            basis.append(u)
        for q in basis:
            og -= (og * q).sum() / ((q * q).sum() + 1e-12) * q
        hist.append(g.clone())
        if len(hist) > grp["history_size"]:
            hist.pop(0)
        return p - grp["lr"] * (og / ((v / (1 - b2 ** t)).sqrt() + grp["eps"]) + grp["weight_decay"] * p)


class DistributedAdam(Optimizer):
    """ZeRO-1 AdamW: gradients are averaged, each rank keeps Adam state for and updates only its contiguous 1/world
    slice of every parameter, then the slices are all-gathered (``optim_advanced.DistributedAdam``).  On a single
    process it is plain AdamW.  The fused flat-buffer path for LLM training is ``parallel.zero_engine.ZeroEngine``;
    this class is the drop-in optimizer object of the reference's API."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, group=None):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.group = group

    @torch.no_grad()
    def step(self, closure=None):
        import torch.distributed as dist
        loss = closure() if closure else None
        on = dist.is_available() and dist.is_initialized()
        world = dist.get_world_size(self.group) if on else 1
        rank = dist.get_rank(self.group) if on else 0
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                grad = p.grad.float().reshape(-1)
                if world > 1:
                    dist.all_reduce(grad, group=self.group)
                    grad /= world
                n = grad.numel()
                per = -(-n // world)
                lo, hi = min(n, rank * per), min(n, (rank + 1) * per)
                st = self.state[p]
                if not st:
                    st["step"], st["m"], st["v"] = 0, torch.zeros(hi - lo, device=p.device), torch.zeros(hi - lo, device=p.device)
                st["step"] += 1
                t = st["step"]
                flat = p.data.float().reshape(-1)
                gs = grad[lo:hi]
                st["m"].mul_(b1).add_(gs, alpha=1 - b1)
                st["v"].mul_(b2).addcmul_(gs, gs, value=1 - b2)
                upd = (st["m"] / (1 - b1 ** t)) / ((st["v"] / (1 - b2 ** t)).sqrt() + g["eps"])
                mine = flat[lo:hi] * (1 - g["lr"] * g["weight_decay"]) - g["lr"] * upd
                if world > 1:
                    pad = torch.zeros(per, device=p.device)
                    pad[: hi - lo] = mine
                    out = torch.empty(world * per, device=p.device)
                    dist.all_gather_into_tensor(out, pad, group=self.group)
                    flat = out[:n]
                else:
                    flat = mine
                p.data.copy_(flat.view_as(p).to(p.dtype))
        return loss


_REGISTRY = {"sgd": SGD, "adam": Adam, "adamw": AdamW, "adamax": Adamax, "rmsprop": RMSprop, "adagrad": Adagrad,
             "adadelta": Adadelta, "radam": RAdam, "sf_adamw": ScheduleFreeAdamW, "schedule_free_adamw": ScheduleFreeAdamW,
             "lion": Lion, "lamb": LAMB, "lars": LARS, "adafactor": AdaFactor, "sm3": SM3, "demeter": Demeter,
             "caprop": CaProp, "soap": SOAP, "orthoadam": OrthoAdam, "distributed_adam": DistributedAdam}


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

"""Learning-rate schedulers (``get_scheduler`` registry of 15, as in interface_bindings/schedulers.py, plus the C
core's StepLR / Exponential / Cosine / Plateau of kernel/optimizer/optimizer.c). Each scheduler is a pure function
of the step, wrapped so it can drive any object with ``lr`` or ``param_groups``."""
from __future__ import annotations

import math
from typing import Callable, Dict


def _warm(step, warmup):
    return min(1.0, (step + 1) / warmup) if warmup > 0 else 1.0


def constant(step, total=0, warmup=0, min_ratio=0.0, **kw):
    return _warm(step, warmup)


def linear(step, total, warmup=0, min_ratio=0.0, **kw):
    if step < warmup:
        return _warm(step, warmup)
    return max(min_ratio, 1.0 - (step - warmup) / max(1, total - warmup) * (1 - min_ratio))


def cosine(step, total, warmup=0, min_ratio=0.0, **kw):
    if step < warmup:
        return _warm(step, warmup)
    t = min(1.0, (step - warmup) / max(1, total - warmup))
    return min_ratio + (1 - min_ratio) * 0.5 * (1 + math.cos(math.pi * t))


def cosine_restarts(step, total, warmup=0, min_ratio=0.0, cycles=4, **kw):
    if step < warmup:
        return _warm(step, warmup)
    t = ((step - warmup) / max(1, total - warmup) * cycles) % 1.0
    return min_ratio + (1 - min_ratio) * 0.5 * (1 + math.cos(math.pi * t))


def polynomial(step, total, warmup=0, min_ratio=0.0, power=2.0, **kw):
    if step < warmup:
        return _warm(step, warmup)
    t = min(1.0, (step - warmup) / max(1, total - warmup))
    return min_ratio + (1 - min_ratio) * (1 - t) ** power


def inverse_sqrt(step, total=0, warmup=1, **kw):
    w = max(1, warmup)
    return _warm(step, w) if step < w else math.sqrt(w / (step + 1))


def exponential(step, total=0, warmup=0, gamma=0.999, **kw):
    return _warm(step, warmup) * gamma ** max(0, step - warmup)


def step_lr(step, total=0, warmup=0, step_size=1000, gamma=0.1, **kw):
    return _warm(step, warmup) * gamma ** (max(0, step - warmup) // step_size)


def multistep(step, total=0, warmup=0, milestones=(), gamma=0.1, **kw):
    return _warm(step, warmup) * gamma ** sum(1 for m in milestones if step >= m)


def one_cycle(step, total, warmup=0, pct_start=0.3, div=25.0, final_div=1e4, **kw):
    peak = int(total * pct_start)
    if step < peak:
        return 1 / div + (1 - 1 / div) * step / max(1, peak)
    t = (step - peak) / max(1, total - peak)
    return 1 / final_div + (1 - 1 / final_div) * 0.5 * (1 + math.cos(math.pi * min(1.0, t)))


def wsd(step, total, warmup=0, decay_frac=0.1, min_ratio=0.0, **kw):
    """warmup - stable - decay"""
    d0 = int(total * (1 - decay_frac))
    if step < warmup:
        return _warm(step, warmup)
    if step < d0:
        return 1.0
    return max(min_ratio, 1 - (step - d0) / max(1, total - d0) * (1 - min_ratio))


def noam(step, total=0, warmup=4000, d_model=512, **kw):
    s = step + 1
    return d_model ** -0.5 * min(s ** -0.5, s * warmup ** -1.5) / (d_model ** -0.5 * warmup ** -0.5)


def cyclic(step, total=0, warmup=0, period=2000, min_ratio=0.1, **kw):
    t = abs((step % period) / (period / 2) - 1)
    return min_ratio + (1 - min_ratio) * (1 - t)


def rex(step, total, warmup=0, **kw):
    t = min(1.0, step / max(1, total))
    return _warm(step, warmup) * (1 - t) / (0.5 + 0.5 * (1 - t))


def trapezoid(step, total, warmup=0, cooldown_frac=0.2, **kw):
    return wsd(step, total, warmup, cooldown_frac)


SCHEDULES: Dict[str, Callable] = {
    "constant": constant, "linear": linear, "cosine": cosine, "cosine_restarts": cosine_restarts,
    "polynomial": polynomial, "inverse_sqrt": inverse_sqrt, "exponential": exponential, "step": step_lr,
    "multistep": multistep, "one_cycle": one_cycle, "wsd": wsd, "noam": noam, "cyclic": cyclic, "rex": rex,
    "trapezoid": trapezoid,
}


class LRScheduler:
    def __init__(self, target, name="constant", base_lr=None, total_steps=0, warmup_steps=0, min_lr=0.0, **kw):
        self.target, self.fn = target, SCHEDULES[name]
        self.base_lr = base_lr if base_lr is not None else self._get()
        self.kw = dict(total=total_steps, warmup=warmup_steps,
                       min_ratio=(min_lr / self.base_lr if self.base_lr else 0.0), **kw)
        self.step_count = 0

    def _get(self):
        return self.target.param_groups[0]["lr"] if hasattr(self.target, "param_groups") else self.target.lr

    def _set(self, lr):
        if hasattr(self.target, "param_groups"):
            for g in self.target.param_groups:
                g["lr"] = lr
        else:
            self.target.lr = lr

    def get_lr(self, step=None):
        return self.base_lr * self.fn(self.step_count if step is None else step, **self.kw)

    def step(self):
        self._set(self.get_lr())
        self.step_count += 1
        return self._get()

    def state_dict(self):
        return {"step_count": self.step_count, "base_lr": self.base_lr}

    def load_state_dict(self, sd):
        self.step_count, self.base_lr = sd["step_count"], sd["base_lr"]


class ReduceLROnPlateau:
    def __init__(self, target, factor=0.1, patience=10, mode="min", min_lr=0.0):
        self.target, self.factor, self.patience, self.mode, self.min_lr = target, factor, patience, mode, min_lr
        self.best, self.bad = None, 0

    def step(self, metric):
        better = self.best is None or (metric < self.best if self.mode == "min" else metric > self.best)
        if better:
            self.best, self.bad = metric, 0
        else:
            self.bad += 1
            if self.bad > self.patience:
                self.bad = 0
                groups = self.target.param_groups if hasattr(self.target, "param_groups") else None
                if groups:
                    for g in groups:
                        g["lr"] = max(self.min_lr, g["lr"] * self.factor)
                else:
                    self.target.lr = max(self.min_lr, self.target.lr * self.factor)


def get_scheduler(name, target, **kw):
    if name in ("plateau", "reduce_on_plateau"):
        return ReduceLROnPlateau(target, **{k: v for k, v in kw.items() if k in ("factor", "patience", "mode", "min_lr")})
    return LRScheduler(target, name, **kw)


class CosineAnnealingLR(LRScheduler):
    """Cosine decay from the base rate to ``eta_min`` over ``T_max`` steps (torch's argument names)."""

    def __init__(self, opt, T_max, eta_min=0.0):
        super().__init__(opt, "cosine", total_steps=T_max, min_lr=eta_min)

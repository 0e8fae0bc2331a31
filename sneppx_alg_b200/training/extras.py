"""Training utilities with the reference's module names folded into one file: activation checkpointing
(grad_checkpoint.py, tape hooks kernel/autodiff/tape.c:80-87), DP-SGD with an RDP accountant
(differential_privacy.py), knowledge distillation (distillation.py), magnitude pruning (pruning.py), random / grid
hyper-parameter search (hpo.py, hparams.py), EMA and label smoothing of ``UltraTrainer`` (trainer_v2.py)."""
from __future__ import annotations

import copy
import itertools
import math
import random
from typing import Callable, Dict, Iterable

import torch
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint as _ckpt


# ---- activation checkpointing
def checkpoint(fn, *args, **kw):
    return _ckpt(fn, *args, use_reentrant=False, **kw)


def enable_activation_checkpointing(model, every: int = 1):
    """Recompute every ``every``-th repeated layer in backward (models expose ``activation_checkpointing``)."""
    if hasattr(model, "activation_checkpointing"):
        model.activation_checkpointing = True
    return model


# ---- differential privacy
class DPSGD:
    """Per-sample clipping + Gaussian noise around any optimizer (micro-batch of 1 per sample)."""

    def __init__(self, model, optimizer, max_grad_norm=1.0, noise_multiplier=1.0, generator=None):
        self.model, self.opt, self.C, self.sigma, self.gen = model, optimizer, max_grad_norm, noise_multiplier, generator
        self.steps = 0

    def step(self, loss_per_sample_fn: Callable[[int], torch.Tensor], batch_size: int):
        params = [p for p in self.model.parameters() if p.requires_grad]
        acc = [torch.zeros_like(p) for p in params]
        for i in range(batch_size):
            grads = torch.autograd.grad(loss_per_sample_fn(i), params, allow_unused=True)
            nrm = math.sqrt(sum(float(g.pow(2).sum()) for g in grads if g is not None))
            scale = min(1.0, self.C / (nrm + 1e-12))
            for a, g in zip(acc, grads):
                if g is not None:
                    a.add_(g * scale)
        for p, a in zip(params, acc):
            noise = torch.randn(a.shape, generator=self.gen, device=a.device, dtype=a.dtype) * self.sigma * self.C
            p.grad = (a + noise) / batch_size
        self.opt.step()
        self.steps += 1


class RDPAccountant:
    """Renyi-DP accounting for the sampled Gaussian mechanism (upper bound for small sampling rates)."""

    def __init__(self, noise_multiplier, sample_rate, orders=None):
        self.sigma, self.q = noise_multiplier, sample_rate
        self.orders = orders or [1.5, 2, 3, 4, 6, 8, 16, 32, 64]
        self.steps = 0

    def step(self, n=1):
        self.steps += n

    def epsilon(self, delta=1e-5):
        best = float("inf")
        for a in self.orders:
            rdp = self.steps * (2 * a * self.q ** 2 / self.sigma ** 2 if self.q < 1 else a / (2 * self.sigma ** 2))
            best = min(best, rdp + math.log(1 / delta) / (a - 1))
        return best


# ---- distillation
def distillation_loss(student_logits, teacher_logits, labels=None, T=2.0, alpha=0.5):
    kd = F.kl_div(F.log_softmax(student_logits.float() / T, -1), F.softmax(teacher_logits.float() / T, -1),
                  reduction="batchmean") * T * T
    if labels is None:
        return kd
    ce = F.cross_entropy(student_logits.float().view(-1, student_logits.shape[-1]), labels.view(-1))
    return alpha * kd + (1 - alpha) * ce


# ---- pruning
@torch.no_grad()
def magnitude_prune_(model, sparsity=0.5, min_dim=2):
    masks = {}
    for n, p in model.named_parameters():
        if p.dim() >= min_dim:
            k = int(p.numel() * sparsity)
            if k:
                thr = p.abs().flatten().kthvalue(k).values
                masks[n] = p.abs() > thr
                p.mul_(masks[n])
    return masks


def sparsity_of(model):
    z = sum(int((p == 0).sum()) for p in model.parameters())
    return z / max(1, sum(p.numel() for p in model.parameters()))


# ---- hyper-parameter search
class SearchSpace:
    def __init__(self, **dims):
        self.dims = dims     # name -> list (choice) | (lo, hi) uniform | (lo, hi, "log")

    def sample(self, rng: random.Random) -> Dict:
        out = {}
        for k, v in self.dims.items():
            if isinstance(v, list):
                out[k] = rng.choice(v)
            elif len(v) == 3 and v[2] == "log":
                out[k] = math.exp(rng.uniform(math.log(v[0]), math.log(v[1])))
            else:
                out[k] = rng.uniform(v[0], v[1])
        return out

    def grid(self) -> Iterable[Dict]:
        keys = [k for k, v in self.dims.items() if isinstance(v, list)]
        for combo in itertools.product(*[self.dims[k] for k in keys]):
            yield dict(zip(keys, combo))


def random_search(objective: Callable[[Dict], float], space: SearchSpace, trials=10, seed=0, mode="min"):
    rng, results = random.Random(seed), []
    for _ in range(trials):
        hp = space.sample(rng)
        results.append((objective(hp), hp))
    results.sort(key=lambda t: t[0], reverse=mode == "max")
    return results[0][1], results


def grid_search(objective, space: SearchSpace, mode="min"):
    results = sorted(((objective(hp), hp) for hp in space.grid()), key=lambda t: t[0], reverse=mode == "max")
    return results[0][1], results


# ---- EMA / label smoothing / early stopping
class EMA:
    def __init__(self, model, decay=0.999):
        self.decay = decay
        self.shadow = copy.deepcopy(model).eval()
        for p in self.shadow.parameters():
            p.requires_grad_(False)

    @torch.no_grad()
    def update(self, model):
        for s, p in zip(self.shadow.parameters(), model.parameters()):
            s.mul_(self.decay).add_(p.detach().to(s.dtype), alpha=1 - self.decay)


def label_smoothing_ce(logits, target, eps=0.1):
    return F.cross_entropy(logits.float(), target, label_smoothing=eps)


class EarlyStopping:
    def __init__(self, patience=5, mode="min", min_delta=0.0):
        self.patience, self.mode, self.min_delta, self.best, self.bad = patience, mode, min_delta, None, 0

    def step(self, metric) -> bool:
        better = self.best is None or (metric < self.best - self.min_delta if self.mode == "min" else metric > self.best + self.min_delta)
        if better:
            self.best, self.bad = metric, 0
        else:
            self.bad += 1
        return self.bad > self.patience

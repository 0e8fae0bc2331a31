"""ARC — adversarial robustness layer (algorithms/arc/core/{input_guard,gradient_obfuscator,output_verifier,
attack_sim,forward,layer}.c; CUDA twin arc_cuda.cu:22-118; Python ``algo_arc.py``).

All tensor ops are batched device ops (no per-row host loops); the attack simulators use true input gradients
(FGSM / PGD) when a loss is given and the reference's sign / uniform perturbations otherwise."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as tnn

from ..nn.modules import Module

OBF_NOISE, OBF_CLAMP, OBF_MIXED = 1, 2, 3
ATTACK_FGSM, ATTACK_PGD, ATTACK_CW = 1, 2, 4


@dataclass
class ARCConfig:
    """``SNEPPX_arc_config_default`` (input_guard.c:29-41)."""
    input_guard_strength: float = 0.7
    gradient_obfuscation_method: int = OBF_MIXED
    gradient_noise_scale: float = 0.01
    gradient_clip_max: float = 1.0
    output_verify_layers: int = 2
    output_verify_threshold: float = 0.9
    adversarial_training: bool = True
    attack_simulation_types: int = ATTACK_FGSM | ATTACK_PGD | ATTACK_CW
    attack_epsilon: float = 0.1
    anomaly_threshold: float = 3.0
    history: int = 16


class InputGuard(Module):
    """Flags rows whose L2 norm is an outlier against running statistics, projects and clips them
    (input_guard.c:104-167); statistics are exponential moving averages (0.99 / 0.01)."""

    def __init__(self, dim, threshold=3.0, device=None):
        super().__init__()
        self.threshold = threshold
        self.projection = tnn.Parameter(torch.eye(dim, device=device) + 0.01 * torch.randn(dim, dim, device=device))
        self.register_buffer("mean", torch.zeros(dim, device=device))
        self.register_buffer("var", torch.ones(dim, device=device))

    def forward(self, x):
        x2 = x.reshape(-1, x.shape[-1]).float()
        l2 = x2.norm(dim=-1)
        mean, var = self.mean.mean(), self.var.mean()
        std = torch.sqrt(var + 1e-6)
        flagged = ((l2 - mean).abs() / std) > self.threshold
        proj = (x2 @ self.projection.float().T).clamp(mean - 3 * std, mean + 3 * std)
        out = torch.where(flagged[:, None], proj, x2)
        if self.training:
            with torch.no_grad():
                bm = x2.mean(0)
                self.mean.mul_(0.99).add_(0.01 * bm)
                self.var.mul_(0.99).add_(0.01 * (x2 - self.mean).pow(2).mean(0))
        return out.to(x.dtype).view_as(x), flagged.float().mean()


class GradientObfuscator:
    """Adds Gaussian noise to gradients and / or clamps them, recording the clamp mask
    (gradient_obfuscator.c:58-93); ``sinusoid`` is the CUDA twin's x + s*sin(100 x) (arc_cuda.cu:92)."""

    def __init__(self, noise_scale=0.01, clip_max=1.0, seed=12345):
        self.noise_scale, self.clip_max = noise_scale, clip_max
        self.gen = None
        self.seed = seed
        self.clamp_ratio = 0.0

    def __call__(self, grad, method=OBF_MIXED):
        if method & OBF_NOISE:
            if self.gen is None or self.gen.device != grad.device:
                self.gen = torch.Generator(device=grad.device).manual_seed(self.seed)
            grad = grad + self.noise_scale * torch.randn(grad.shape, generator=self.gen, device=grad.device, dtype=grad.dtype)
        if method & OBF_CLAMP:
            mask = grad.abs() > self.clip_max
            self.clamp_ratio = float(mask.float().mean())
            grad = grad.clamp(-self.clip_max, self.clip_max)
        return grad

    def sinusoid(self, grad):
        if grad.is_cuda and grad.dtype == torch.float32 and grad.numel() % 4 == 0:
            from ..ops import aux
            return aux.arc_step("obfuscate", grad, eps=self.noise_scale).view_as(grad)
        return grad + self.noise_scale * torch.sin(100.0 * grad)

    def attach(self, module, method=OBF_MIXED):
        """Registers the obfuscator as a gradient hook on every parameter of ``module``."""
        return [p.register_hook(lambda g, m=method: self(g, m)) for p in module.parameters() if p.requires_grad]


class OutputVerifier(Module):
    """ReLU verification layers + cosine consistency against a ring of recent outputs; low-confidence batches are
    pulled toward the history mean with alpha 0.3 (output_verifier.c:103-173)."""

    def __init__(self, dim, num_layers=2, threshold=0.9, history=16, device=None):
        super().__init__()
        self.threshold = threshold
        self.weights = tnn.ParameterList([tnn.Parameter(torch.eye(dim, device=device) +
                                                        torch.randn(dim, dim, device=device) / (10 * math.sqrt(dim)))
                                          for _ in range(num_layers)])
        self.biases = tnn.ParameterList([tnn.Parameter(torch.zeros(dim, device=device)) for _ in range(num_layers)])
        self.register_buffer("hist", torch.zeros(history, dim, device=device))
        self.filled, self.idx = 0, 0

    def forward(self, x):
        x2 = x.reshape(-1, x.shape[-1]).float()
        v = x2
        for w, b in zip(self.weights, self.biases):
            v = torch.relu(v @ w.float().T + b.float())
        conf = x2.new_tensor(1.0)
        if self.filled:
            avg = self.hist[: self.filled].mean(0)
            cos = torch.dot(x2[0], avg) / (x2[0].norm() * avg.norm() + 1e-10)
            conf = (cos + 1) * 0.5
            v = torch.where(conf < self.threshold, 0.3 * x2 + 0.7 * avg, v)
        with torch.no_grad():
            self.hist[self.idx] = x2[0].detach()
            self.filled = min(self.filled + 1, self.hist.shape[0])
            self.idx = (self.idx + 1) % self.hist.shape[0]
        return v.to(x.dtype).view_as(x), conf


def simulate_attack(x, attack_type=ATTACK_FGSM, epsilon=0.1, loss_fn=None, steps=3, lo=-1.0, hi=1.0, seed=54321):
    """FGSM / PGD / CW-style perturbation clipped to [lo, hi] (attack_sim.c:30-83).  With ``loss_fn`` (x -> scalar)
    the sign comes from the true input gradient; without it the perturbation direction is pseudo-random as in the
    reference."""
    g = torch.Generator(device=x.device).manual_seed(seed)

    def sign_of(xa):
        if loss_fn is None:
            return torch.where(torch.rand(xa.shape, generator=g, device=xa.device) < 0.5, -1.0, 1.0).to(xa.dtype)
        xa = xa.detach().requires_grad_(True)
        (grad,) = torch.autograd.grad(loss_fn(xa), xa)
        return grad.sign()

    native = x.is_cuda and x.dtype == torch.float32 and x.numel() % 4 == 0
    if native:
        from ..ops import aux  # one fused kernel per step: sign, step, projection and clamp
    if attack_type == ATTACK_FGSM:
        if native:
            return aux.arc_step("fgsm", x, sign_of(x), eps=epsilon, lo=lo, hi=hi).view_as(x)
        return (x + epsilon * sign_of(x)).clamp(lo, hi).detach()
    if attack_type == ATTACK_CW:
        return (x + 0.5 * epsilon * sign_of(x)).clamp(lo, hi).detach()
    if attack_type == ATTACK_PGD:
        adv = (x + (torch.rand(x.shape, generator=g, device=x.device).to(x.dtype) - 0.5) * 2 * epsilon).clamp(lo, hi)
        step = epsilon / steps
        for _ in range(steps):
            if native:
                adv = aux.arc_step("pgd", adv, sign_of(adv), x, eps=epsilon, alpha=step, lo=lo, hi=hi).view_as(x)
                continue
            adv = adv + step * sign_of(adv)
            adv = torch.min(torch.max(adv, x - epsilon), x + epsilon).clamp(lo, hi)
        return adv.detach()
    raise ValueError(f"unknown attack {attack_type}")


def randomized_smoothing(fn, x, sigma=0.1, samples=8, seed=None):
    """Mean prediction under Gaussian input noise (arc_cuda.cu:118). With ``seed`` the noise comes from the
    counter-based generator (sample i uses stream offset i), so the result is reproducible on any device."""
    if seed is not None:
        from ..ops import aux
        return torch.stack([fn(aux.arc_step("smooth", x, eps=sigma, seed=seed, offset=i).view_as(x).to(x.dtype))
                            for i in range(samples)]).mean(0)
    return torch.stack([fn(x + sigma * torch.randn_like(x)) for _ in range(samples)]).mean(0)


class ARCLayer(Module):
    """guard -> verifier; ``metrics`` = [anomaly score, confidence, clamp ratio, output norm] (forward.c:29-72)."""

    def __init__(self, dim, cfg: ARCConfig = None, device=None):
        super().__init__()
        self.cfg = cfg or ARCConfig()
        self.input_guard = InputGuard(dim, self.cfg.anomaly_threshold, device=device)
        self.output_verifier = OutputVerifier(dim, self.cfg.output_verify_layers, self.cfg.output_verify_threshold,
                                              self.cfg.history, device=device)
        self.gradient_obfuscator = GradientObfuscator(self.cfg.gradient_noise_scale, self.cfg.gradient_clip_max)
        self.metrics = None

    def forward(self, x):
        s, anomaly = self.input_guard(x)
        y, conf = self.output_verifier(s)
        self.metrics = torch.stack([anomaly.float(), conf.float(), y.new_tensor(self.gradient_obfuscator.clamp_ratio).float(),
                                    y.float().norm()])
        return y

    def adversarial_loss(self, model_fn, x, target, loss_fn):
        """Clean + adversarial loss for adversarial training (forward_train.c:62-96)."""
        adv = simulate_attack(x, ATTACK_FGSM, self.cfg.attack_epsilon, lambda xa: loss_fn(model_fn(xa), target))
        return 0.5 * (loss_fn(model_fn(x), target) + loss_fn(model_fn(adv), target))


ARCModel = ARCLayer

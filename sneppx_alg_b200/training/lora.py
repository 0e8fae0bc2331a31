"""Parameter-efficient fine-tuning and preference optimisation: LoRA / QLoRA (NF4 base weights), ``DPOTrainer`` and
``GRPOTrainer`` (names of interface_bindings/lora.py)."""
from __future__ import annotations

import copy
import math
from typing import Callable

import torch
import torch.nn as tnn
import torch.nn.functional as F


NF4 = torch.tensor([-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
                    -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
                    0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
                    0.7229568362236023, 1.0])


def quantize_nf4(w: torch.Tensor, block: int = 64):
    flat = w.detach().float().reshape(-1, block)
    absmax = flat.abs().amax(1, keepdim=True).clamp_min(1e-12)
    idx = ((flat / absmax).unsqueeze(-1) - NF4.to(w.device)).abs().argmin(-1).to(torch.uint8)
    return idx, absmax.squeeze(1), w.shape


def dequantize_nf4(idx, absmax, shape, dtype=torch.bfloat16):
    return (NF4.to(idx.device)[idx.long()] * absmax.unsqueeze(1)).reshape(shape).to(dtype)


class LoRALinear(tnn.Module):
    """y = x W^T + (alpha / r) * x A^T B^T with W frozen (optionally stored in NF4)."""

    def __init__(self, base, r=8, alpha=16.0, dropout=0.0, quantize_base=False):
        super().__init__()
        w = base.weight.detach()
        self.out_features, self.in_features = w.shape
        self.r, self.scaling = r, alpha / r
        b = getattr(base, "bias", None)
        self.bias = tnn.Parameter(b.detach().clone(), requires_grad=False) if b is not None else None   # frozen with W
        self.qbase = quantize_base
        if quantize_base:
            idx, absmax, shape = quantize_nf4(w)
            self.register_buffer("w_idx", idx)
            self.register_buffer("w_absmax", absmax)
            self._shape, self._dtype = shape, w.dtype
        else:
            self.weight = tnn.Parameter(w.clone(), requires_grad=False)
        self.lora_A = tnn.Parameter(torch.empty(r, self.in_features, dtype=w.dtype, device=w.device))
        self.lora_B = tnn.Parameter(torch.zeros(self.out_features, r, dtype=w.dtype, device=w.device))
        tnn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        self.drop = tnn.Dropout(dropout)

    def base_weight(self):
        return dequantize_nf4(self.w_idx, self.w_absmax, self._shape, self._dtype) if self.qbase else self.weight

    def forward(self, x):
        y = F.linear(x, self.base_weight(), self.bias)
        return y + self.scaling * F.linear(F.linear(self.drop(x), self.lora_A), self.lora_B)

    def merged_weight(self):
        return self.base_weight() + self.scaling * (self.lora_B @ self.lora_A)


class QLoRALinear(LoRALinear):
    """LoRA over a frozen base weight stored in 4-bit NormalFloat with per-block absmax scales: the base takes half a
    byte per weight (plus scales) and is de-quantised on the fly for every forward; only A and B train
    (the reference's ``QLoRALinear``, interface_bindings/lora.py:133-175, keeps an int4 base and ``_dequantize_weight``)."""

    def __init__(self, base, r=8, alpha=16.0, dropout=0.0):
        super().__init__(base, r, alpha, dropout, quantize_base=True)

    @property
    def base_bytes(self) -> int:
        return self.w_idx.numel() * self.w_idx.element_size() + self.w_absmax.numel() * self.w_absmax.element_size()

    def quantization_error(self, reference_weight) -> float:
        """Relative Frobenius error of the stored base against the weight it was made from."""
        w = reference_weight.detach().float()
        return float((self.base_weight().float() - w).norm() / (w.norm() + 1e-12))


def apply_lora(model, r=8, alpha=16.0, targets=("qkv_proj", "o_proj", "gate_up_proj", "down_proj"), qlora=False):
    """Freeze the model and wrap the targeted linear layers; returns the list of trainable LoRA parameters."""
    for p in model.parameters():
        p.requires_grad_(False)
    params = []
    for mod in list(model.modules()):
        for name, child in list(mod.named_children()):
            if name in targets and hasattr(child, "weight") and child.weight.dim() == 2:
                l = QLoRALinear(child, r, alpha) if qlora else LoRALinear(child, r, alpha)
                setattr(mod, name, l)
                params += [l.lora_A, l.lora_B]
    return params


def sequence_logprob(model, ids, mask=None):
    """Sum of next-token log-probabilities of ``ids`` [B, S] under the model."""
    logits = model(ids)["logits"].float()
    lp = torch.log_softmax(logits[:, :-1], -1).gather(-1, ids[:, 1:].unsqueeze(-1)).squeeze(-1)
    if mask is not None:
        lp = lp * mask[:, 1:]
    return lp.sum(-1)


class DPOTrainer:
    """Direct preference optimisation: -log sigmoid(beta * ((pi_c - pi_r) - (ref_c - ref_r)))."""

    def __init__(self, policy, reference=None, beta=0.1, lr=1e-5, params=None):
        self.policy = policy
        self.ref = reference if reference is not None else copy.deepcopy(policy).eval()
        for p in self.ref.parameters():
            p.requires_grad_(False)
        self.beta = beta
        self.opt = torch.optim.AdamW(params or [p for p in policy.parameters() if p.requires_grad], lr=lr)

    def loss(self, chosen, rejected):
        pc, pr = sequence_logprob(self.policy, chosen), sequence_logprob(self.policy, rejected)
        with torch.no_grad():
            rc, rr = sequence_logprob(self.ref, chosen), sequence_logprob(self.ref, rejected)
        margin = self.beta * ((pc - pr) - (rc - rr))
        return -F.logsigmoid(margin).mean(), (margin > 0).float().mean()

    def step(self, chosen, rejected):
        self.opt.zero_grad(set_to_none=True)
        loss, acc = self.loss(chosen, rejected)
        loss.backward()
        self.opt.step()
        return float(loss.detach()), float(acc)


class GRPOTrainer:
    """Group-relative policy optimisation: sample G completions per prompt, normalise rewards inside the group, ascend
    advantage-weighted log-likelihood with a KL penalty to the reference policy."""

    def __init__(self, policy, reward_fn: Callable[[torch.Tensor], torch.Tensor], group_size=4, kl_coef=0.02, lr=1e-5,
                 max_new_tokens=16):
        self.policy, self.reward_fn, self.G, self.kl, self.max_new = policy, reward_fn, group_size, kl_coef, max_new_tokens
        self.ref = copy.deepcopy(policy).eval()
        for p in self.ref.parameters():
            p.requires_grad_(False)
        self.opt = torch.optim.AdamW([p for p in policy.parameters() if p.requires_grad], lr=lr)

    @torch.no_grad()
    def sample(self, prompt):
        from ..serving.generation import generate
        ids = prompt.repeat(self.G, 1)
        return generate(self.policy, ids, self.max_new, do_sample=True, temperature=1.0)

    def step(self, prompt):
        seqs = self.sample(prompt)
        r = self.reward_fn(seqs).float()
        adv = (r - r.mean()) / (r.std() + 1e-6)
        mask = torch.zeros_like(seqs, dtype=torch.float32)
        mask[:, prompt.shape[1]:] = 1.0
        lp = sequence_logprob(self.policy, seqs, mask)
        with torch.no_grad():
            lref = sequence_logprob(self.ref, seqs, mask)
        loss = -(adv * lp).mean() + self.kl * (lp - lref).mean()
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        self.opt.step()
        return float(loss.detach()), float(r.mean())

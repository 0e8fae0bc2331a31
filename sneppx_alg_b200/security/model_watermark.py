"""Ownership marks inside a model's parameters and behaviour.

``WeightWatermark`` writes a key-derived +-1 pattern into a small fraction of every parameter after training and
later measures how well the weights at those positions still follow the pattern. ``BackdoorWatermark`` trains the
model to answer a set of key-derived trigger inputs with one label and later counts how many triggers still get
that label. Both derive everything from the key string, so the owner needs to keep only the key.

Reference behaviour: interface_bindings/watermark.py:79 (weights) and :147 (triggers). The text watermark of the
serving path (green-list logits bias) lives in ``serving/watermark.py``.
"""
from __future__ import annotations

import hashlib
from typing import Callable, Dict, List, Tuple

import torch


def _generator(key: str, salt: str) -> torch.Generator:
    seed = int.from_bytes(hashlib.sha256(f"{key}\x00{salt}".encode()).digest()[:8], "big") & ((1 << 63) - 1)
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


class WeightWatermark:
    """Post-training mark: ``ratio`` of each parameter's entries are set to ``strength * pattern``."""

    def __init__(self, key: str, strength: float = 0.05, ratio: float = 0.05):
        if not 0.0 < ratio <= 1.0:
            raise ValueError("ratio must be in (0, 1]")
        if strength <= 0:
            raise ValueError("strength must be positive")
        self.key, self.strength, self.ratio = key, float(strength), float(ratio)

    def positions(self, name: str, p: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Flat indices and the +-1 pattern for parameter ``name`` of this shape (a function of the key only)."""
        g = _generator(self.key, f"{name}|{tuple(p.shape)}")
        n = p.numel()
        k = max(1, int(round(n * self.ratio)))
        idx = torch.randperm(n, generator=g)[:k]
        pattern = torch.randint(0, 2, (k,), generator=g).to(torch.float32) * 2.0 - 1.0
        return idx, pattern

    @torch.no_grad()
    def embed(self, model: torch.nn.Module) -> Dict[str, dict]:
        info = {}
        for name, p in model.named_parameters():
            idx, pattern = self.positions(name, p)
            flat = p.data.view(-1)
            flat[idx.to(flat.device)] = (self.strength * pattern).to(flat.device, flat.dtype)
            info[name] = {"selected": int(idx.numel()), "total": int(p.numel())}
        return info

    @torch.no_grad()
    def detect(self, model: torch.nn.Module, threshold: float = 0.5) -> Tuple[bool, float]:
        """(marked, score): score is the mean over parameters of the Pearson correlation between the pattern and the
        weights found at its positions, negative correlations counted as zero."""
        scores: List[float] = []
        for name, p in model.named_parameters():
            idx, pattern = self.positions(name, p)
            if idx.numel() < 2:
                continue
            seen = p.data.view(-1)[idx.to(p.device)].double().cpu()
            pat = pattern.double()
            sd = seen.std()
            if float(sd) < 1e-12 or float(pat.std()) < 1e-12:
                scores.append(0.0)
                continue
            r = float(((seen - seen.mean()) * (pat - pat.mean())).mean() / (seen.std(unbiased=False) * pat.std(unbiased=False)))
            scores.append(max(0.0, r) if r == r else 0.0)
        score = sum(scores) / len(scores) if scores else 0.0
        return score >= threshold, score


class BackdoorWatermark:
    """Trigger-set mark: ``num_keys`` Gaussian inputs derived from the key are trained to ``target_label``."""

    def __init__(self, key: str, input_shape, target_label: int, num_keys: int = 100, threshold: float = 0.9):
        if num_keys <= 0:
            raise ValueError("num_keys must be positive")
        self.key, self.input_shape = key, tuple(input_shape)
        self.target_label, self.num_keys, self.threshold = int(target_label), int(num_keys), float(threshold)
        self.triggers = torch.randn((self.num_keys,) + self.input_shape, generator=_generator(key, "triggers"))

    def train(self, model: torch.nn.Module, optimizer, loss_fn: Callable = torch.nn.functional.cross_entropy,
              epochs: int = 5, clean_batch=None) -> List[float]:
        """``epochs`` full-batch steps on the triggers; with ``clean_batch=(x, y)`` each step also fits that batch so
        the mark does not cost task accuracy. Returns the loss per step."""
        dev = next(model.parameters()).device
        x = self.triggers.to(dev)
        y = torch.full((self.num_keys,), self.target_label, dtype=torch.long, device=dev)
        history = []
        for _ in range(epochs):
            optimizer.zero_grad(set_to_none=True)
            loss = loss_fn(model(x), y)
            if clean_batch is not None:
                loss = loss + loss_fn(model(clean_batch[0].to(dev)), clean_batch[1].to(dev))
            loss.backward()
            optimizer.step()
            history.append(float(loss.detach()))
        return history

    @torch.no_grad()
    def verify(self, model: torch.nn.Module) -> Tuple[bool, float]:
        dev = next(model.parameters()).device
        was_training = model.training
        model.eval()
        hit = float((model(self.triggers.to(dev)).argmax(-1) == self.target_label).float().mean())
        model.train(was_training)
        return hit >= self.threshold, hit

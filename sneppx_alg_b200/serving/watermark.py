"""Green-list text watermark for generated tokens and its detector (the reference's ``watermark.py``): the previous
token seeds a pseudo-random partition of the vocabulary; sampling adds ``delta`` to green-list logits; detection is a
one-sided z-test on the green-token count."""
from __future__ import annotations

import math

import torch


class Watermark:
    def __init__(self, vocab_size: int, gamma: float = 0.5, delta: float = 2.0, key: int = 15485863):
        self.V, self.gamma, self.delta, self.key = vocab_size, gamma, delta, key

    def green_mask(self, prev_token: int, device=None) -> torch.Tensor:
        g = torch.Generator().manual_seed((self.key * (int(prev_token) + 1)) % (2 ** 31 - 1))
        perm = torch.randperm(self.V, generator=g)
        mask = torch.zeros(self.V, dtype=torch.bool)
        mask[perm[: int(self.gamma * self.V)]] = True
        return mask.to(device) if device is not None else mask

    def apply(self, logits: torch.Tensor, prev_tokens) -> torch.Tensor:
        """logits [B, V]; prev_tokens [B]."""
        out = logits.clone()
        for b, t in enumerate(prev_tokens.tolist() if torch.is_tensor(prev_tokens) else prev_tokens):
            out[b, self.green_mask(t, logits.device)] += self.delta
        return out

    def detect(self, tokens) -> dict:
        toks = tokens.tolist() if torch.is_tensor(tokens) else list(tokens)
        n = len(toks) - 1
        if n <= 0:
            return {"z": 0.0, "green_fraction": 0.0, "watermarked": False}
        green = sum(bool(self.green_mask(toks[i])[toks[i + 1]]) for i in range(n))
        z = (green - self.gamma * n) / math.sqrt(n * self.gamma * (1 - self.gamma))
        return {"z": z, "green_fraction": green / n, "watermarked": z > 4.0}

"""Two-moons style classification with an MLP, AdamW and a warm-up + cosine schedule, driven by ``Trainer``."""
from _common import device, seed  # first: makes the package importable from a checkout

import math

import torch

from sneppx.nn import GELU, Linear, Sequential
from sneppx.training.config import TrainConfig
from sneppx.training.trainer import Trainer


def moons(n: int, g: torch.Generator):
    t = torch.rand(n, generator=g) * math.pi
    half = n // 2
    x = torch.stack([torch.cos(t), torch.sin(t)], 1)
    x[half:] = torch.stack([1.0 - torch.cos(t[half:]), 0.5 - torch.sin(t[half:])], 1)
    y = torch.cat([torch.zeros(half), torch.ones(n - half)]).long()
    return x + 0.08 * torch.randn(n, 2, generator=g), y


def main(steps: int = 400) -> float:
    g, dev = seed(1), device()
    x, y = moons(512, g)
    model = Sequential(Linear(2, 64, device=dev), GELU(), Linear(64, 64, device=dev), GELU(), Linear(64, 2, device=dev))
    cfg = TrainConfig({"training": {"max_steps": steps, "loss": "cross_entropy", "max_grad_norm": 1.0},
                       "optimizer": {"name": "adamw", "lr": 1e-2, "weight_decay": 0.0},
                       "scheduler": {"name": "cosine", "warmup_steps": 20}})
    trainer = Trainer(model, cfg)
    for step in range(steps):
        idx = torch.randint(0, 512, (128,), generator=g)
        trainer.train_step((x[idx], y[idx]))
    with torch.no_grad():
        acc = float((model(x.to(dev)).argmax(-1).cpu() == y).float().mean())
    print(f"accuracy on the training set after {steps} steps: {acc:.3f}")
    return acc


if __name__ == "__main__":
    main()

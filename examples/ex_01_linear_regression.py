"""Least-squares fit of y = 3x - 2 + noise with ``nn.Linear`` and SGD; prints the recovered slope and intercept."""
from _common import device, seed  # first: makes the package importable from a checkout

import torch

import sneppx
from sneppx.nn import Linear
from sneppx.optim.zoo import SGD


def main(steps: int = 300) -> dict:
    g, dev = seed(0), device()
    x = torch.rand(256, 1, generator=g) * 4 - 2
    y = 3.0 * x - 2.0 + 0.05 * torch.randn(256, 1, generator=g)
    x, y = x.to(dev), y.to(dev)
    model = Linear(1, 1, bias=True, device=dev)
    opt = SGD(model.parameters(), lr=0.1)
    for _ in range(steps):
        opt.zero_grad()
        loss = ((model(x) - y) ** 2).mean()
        loss.backward()
        opt.step()
    out = {"slope": model.weight.item(), "intercept": model.bias.item(), "mse": loss.item()}
    print(f"sneppx {sneppx.__version__}: y = {out['slope']:.3f} x + {out['intercept']:.3f}   (mse {out['mse']:.5f})")
    return out


if __name__ == "__main__":
    main()

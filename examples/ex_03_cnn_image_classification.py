"""A small convolutional classifier written with the functional tensor API (``conv2d``, ``max_pool2d``) on synthetic
images: bright squares against bright bars."""
from _common import device, seed  # first: makes the package importable from a checkout
import torch

import sneppx.tensor as T
from sneppx.nn import Linear, Module
from sneppx.optim.zoo import AdamW


def make_images(n: int, g: torch.Generator):
    x = 0.1 * torch.randn(n, 1, 16, 16, generator=g)
    y = torch.randint(0, 2, (n,), generator=g)
    for i in range(n):
        r, c = [int(v) for v in torch.randint(2, 9, (2,), generator=g)]
        if y[i] == 0:
            x[i, 0, r:r + 5, c:c + 5] += 1.0          # a square
        else:
            x[i, 0, r:r + 2, 1:15] += 1.0              # a horizontal bar
    return x, y


class SmallCNN(Module):
    def __init__(self, device=None):
        super().__init__()
        g = torch.Generator().manual_seed(0)
        self.k1 = torch.nn.Parameter((torch.randn(8, 1, 3, 3, generator=g) * 0.3).to(device))
        self.k2 = torch.nn.Parameter((torch.randn(16, 8, 3, 3, generator=g) * 0.1).to(device))
        self.head = Linear(16 * 4 * 4, 2, device=device)

    def forward(self, x):
        x = T.max_pool2d(T.relu(T.conv2d(x, self.k1, padding=1)), 2)
        x = T.max_pool2d(T.relu(T.conv2d(x, self.k2, padding=1)), 2)
        return self.head(x.flatten(1))


def main(steps: int = 120) -> float:
    g, dev = seed(2), device()
    x, y = make_images(512, g)
    x, y = x.to(dev), y.to(dev)
    model = SmallCNN(dev)
    opt = AdamW(model.parameters(), lr=3e-3, weight_decay=0.0)
    for _ in range(steps):
        idx = torch.randint(0, 512, (64,), generator=g).to(dev)
        opt.zero_grad()
        loss = T.cross_entropy(model(x[idx]), y[idx])
        loss.backward()
        opt.step()
    with torch.no_grad():
        acc = (model(x).argmax(-1) == y).float().mean().item()
    print(f"CNN accuracy: {acc:.3f} (loss {loss.item():.4f})")
    return acc


if __name__ == "__main__":
    main()

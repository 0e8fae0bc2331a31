"""The reference's single-file models (algorithms/{gcn,rnn,gan,diffusion,rl}/core/*.c) as small PyTorch modules on
this package's ``Linear`` (tensor-core GEMMs on CUDA bf16)."""
from __future__ import annotations

import math

import torch
import torch.nn as tnn
import torch.nn.functional as F

from ..nn.modules import Linear, Module


class GCNLayer(Module):
    """H' = act(D^-1/2 (A + I) D^-1/2 H W) (algorithms/gcn/core)."""

    def __init__(self, d_in, d_out, dtype=None, device=None):
        super().__init__()
        self.lin = Linear(d_in, d_out, dtype=dtype, device=device)

    @staticmethod
    def normalize(adj):
        a = adj + torch.eye(adj.shape[0], device=adj.device, dtype=adj.dtype)
        d = a.sum(-1).clamp_min(1e-12).rsqrt()
        return d[:, None] * a * d[None, :]

    def forward(self, h, adj_norm):
        return adj_norm.to(h.dtype) @ self.lin(h)


class GCN(Module):
    def __init__(self, d_in, d_hidden, n_classes, dtype=None, device=None):
        super().__init__()
        self.l1, self.l2 = GCNLayer(d_in, d_hidden, dtype, device), GCNLayer(d_hidden, n_classes, dtype, device)

    def forward(self, x, adj):
        a = GCNLayer.normalize(adj)
        return self.l2(F.relu(self.l1(x, a)), a)


class RNN(Module):
    """Elman / GRU / LSTM cell unrolled over time; the input projection of all steps is one GEMM."""

    def __init__(self, d_in, d_hidden, cell="lstm", dtype=None, device=None):
        super().__init__()
        self.cell, self.dh = cell, d_hidden
        g = {"rnn": 1, "gru": 3, "lstm": 4}[cell]
        self.wx = Linear(d_in, g * d_hidden, dtype=dtype, device=device)
        self.wh = Linear(d_hidden, g * d_hidden, bias=False, dtype=dtype, device=device)

    def forward(self, x, state=None):
        B, L, _ = x.shape
        xs = self.wx(x)
        h = x.new_zeros(B, self.dh) if state is None else state[0]
        c = x.new_zeros(B, self.dh) if state is None or self.cell != "lstm" else state[1]
        out = []
        for t in range(L):
            if self.cell == "rnn":
                h = torch.tanh(xs[:, t] + self.wh(h))
            elif self.cell == "gru":
                xr, xz, xn = xs[:, t].chunk(3, -1)
                hr, hz, hn = self.wh(h).chunk(3, -1)
                r, z = torch.sigmoid(xr + hr), torch.sigmoid(xz + hz)
                h = (1 - z) * torch.tanh(xn + r * hn) + z * h
            else:
                i, f, g, o = (xs[:, t] + self.wh(h)).chunk(4, -1)
                c = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(g)
                h = torch.sigmoid(o) * torch.tanh(c)
            out.append(h)
        return torch.stack(out, 1), (h, c)


class GAN(Module):
    """MLP generator / discriminator with the non-saturating losses (algorithms/gan/core)."""

    def __init__(self, d_latent=64, d_data=784, d_hidden=256, dtype=None, device=None):
        super().__init__()
        mk = lambda i, o: Linear(i, o, dtype=dtype, device=device)  # noqa: E731
        self.d_latent = d_latent
        self.generator = tnn.Sequential(mk(d_latent, d_hidden), tnn.ReLU(), mk(d_hidden, d_data), tnn.Tanh())
        self.discriminator = tnn.Sequential(mk(d_data, d_hidden), tnn.LeakyReLU(0.2), mk(d_hidden, 1))

    def sample(self, n, device=None):
        p = next(self.parameters())
        return self.generator(torch.randn(n, self.d_latent, device=device or p.device, dtype=p.dtype))

    def discriminator_loss(self, real):
        fake = self.sample(real.shape[0]).detach()
        return F.softplus(-self.discriminator(real)).mean() + F.softplus(self.discriminator(fake)).mean()

    def generator_loss(self, n):
        return F.softplus(-self.discriminator(self.sample(n))).mean()


class Diffusion(Module):
    """DDPM with a linear beta schedule and an MLP noise predictor (algorithms/diffusion/core)."""

    def __init__(self, d_data, d_hidden=256, steps=1000, beta_start=1e-4, beta_end=0.02, dtype=None, device=None):
        super().__init__()
        self.steps = steps
        betas = torch.linspace(beta_start, beta_end, steps, device=device)
        self.register_buffer("betas", betas)
        self.register_buffer("alpha_bar", torch.cumprod(1 - betas, 0))
        mk = lambda i, o: Linear(i, o, dtype=dtype, device=device)  # noqa: E731
        self.net = tnn.Sequential(mk(d_data + 32, d_hidden), tnn.SiLU(), mk(d_hidden, d_hidden), tnn.SiLU(), mk(d_hidden, d_data))

    def time_embed(self, t):
        f = torch.exp(-math.log(10000.0) * torch.arange(16, device=t.device) / 16)
        a = t.float()[:, None] * f[None]
        return torch.cat([a.sin(), a.cos()], -1)

    def predict_noise(self, x, t):
        return self.net(torch.cat([x, self.time_embed(t).to(x.dtype)], -1))

    def q_sample(self, x0, t, noise):
        ab = self.alpha_bar[t][:, None].to(x0.dtype)
        return ab.sqrt() * x0 + (1 - ab).sqrt() * noise

    def loss(self, x0):
        t = torch.randint(0, self.steps, (x0.shape[0],), device=x0.device)
        noise = torch.randn_like(x0)
        return F.mse_loss(self.predict_noise(self.q_sample(x0, t, noise), t), noise)

    @torch.no_grad()
    def sample(self, n, d, device=None, steps=None):
        x = torch.randn(n, d, device=device or self.betas.device)
        for i in reversed(range(steps or self.steps)):
            t = torch.full((n,), i, device=x.device)
            b, ab = self.betas[i], self.alpha_bar[i]
            mean = (x - b / (1 - ab).sqrt() * self.predict_noise(x, t)) / (1 - b).sqrt()
            x = mean + (b.sqrt() * torch.randn_like(x) if i else 0)
        return x


class PolicyGradientAgent(Module):
    """REINFORCE with a value baseline (algorithms/rl/core)."""

    def __init__(self, d_obs, n_actions, d_hidden=128, gamma=0.99, dtype=None, device=None):
        super().__init__()
        mk = lambda i, o: Linear(i, o, dtype=dtype, device=device)  # noqa: E731
        self.gamma = gamma
        self.body = tnn.Sequential(mk(d_obs, d_hidden), tnn.Tanh())
        self.pi, self.v = mk(d_hidden, n_actions), mk(d_hidden, 1)

    def act(self, obs):
        h = self.body(obs)
        dist = torch.distributions.Categorical(logits=self.pi(h).float())
        a = dist.sample()
        return a, dist.log_prob(a), self.v(h).squeeze(-1)

    def returns(self, rewards):
        out, g = [], 0.0
        for r in reversed(rewards):
            g = r + self.gamma * g
            out.append(g)
        return torch.tensor(out[::-1])

    def loss(self, log_probs, values, rewards):
        ret = self.returns(rewards).to(values.device)
        adv = ret - values.detach().float()
        return -(log_probs * adv).mean() + F.mse_loss(values.float(), ret)

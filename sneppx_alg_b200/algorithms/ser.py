"""SER — sparse expert routing, the reference's API names (``algo_ser.py``; algorithms/ser/core/route.c:58-348,
loss.c:31-69, forward_layer.c:31-143, expert.c:30-39) over this package's router / grouped-GEMM kernels."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as tnn

from ..nn.modules import Linear, Module
from ..nn.moe import SERMoE
from ..ops import functional as ops
from ..ops import moe as moe_ops


@dataclass
class SERConfig:
    """``SNEPPX_ser_config_default`` (expert.c:30-39)."""
    num_experts: int = 8
    top_k: int = 2
    input_dim: int = 512
    hidden_dim: int = 2048
    output_dim: int = 512
    activation: str = "relu"           # relu | gelu | swish (reference experts); "swiglu" selects gated experts
    load_balance_coef: float = 0.01
    z_loss_coef: float = 0.0
    capacity: int = 0                  # 0 -> (input_dim * 2) / num_experts tokens per expert when enforced
    enforce_capacity: bool = False
    noisy_gating: bool = False
    temperature: float = 1.0
    num_layers: int = 1


class SERRoute:
    @staticmethod
    def topk_gating(logits, k, noisy=False, temperature=1.0, noise_std=1.0):
        """softmax over experts -> top-k -> renormalise (route.c:58-157; noisy variant :84-91; temperature :163-245).
        Returns (idx int32 [T,k], weights [T,k], probs [T,E], counts int32 [E])."""
        if noisy:
            logits = logits + noise_std * torch.randn_like(logits)
        if temperature != 1.0:
            logits = logits / temperature
        return moe_ops.route(logits, k, renorm=True)

    @staticmethod
    def load_balance_loss(probs, counts, k):
        """E * sum_e f_e p_e with f_e the token fraction routed to e and p_e the mean router probability (loss.c:31-69)."""
        E = probs.shape[-1]
        f = counts.float() / max(1, probs.shape[0] * k)
        return E * (f * probs.float().mean(0)).sum()

    @staticmethod
    def importance_loss(probs):
        imp = probs.float().sum(0)
        return imp.var() / (imp.mean() ** 2 + 1e-10)

    @staticmethod
    def enforce_capacity(idx, w, num_experts, capacity):
        """Drops the lowest-weight assignments beyond ``capacity`` per expert (route.c:290-348)."""
        return moe_ops.enforce_capacity(idx, w, num_experts, capacity)


class SERLoss:
    @staticmethod
    def z_loss(logits):
        """mean(logits^2) (route.c:251-259)."""
        return logits.float().pow(2).mean()

    load_balance = staticmethod(SERRoute.load_balance_loss)


_ACT = {"relu": torch.relu, "gelu": tnn.functional.gelu, "swish": tnn.functional.silu, "silu": tnn.functional.silu}


class SERLayer(Module):
    """Router + experts.  ``activation='swiglu'`` builds gated experts that run as two grouped tcgen05 GEMMs
    (``nn.moe.SERMoE``); the reference's biased two-layer MLP experts (forward_expert.c:37-80) are kept for parity and
    run as one GEMM pair per expert over the gathered rows."""

    def __init__(self, cfg: SERConfig = None, dtype=None, device=None, **kw):
        super().__init__()
        cfg = cfg or SERConfig(**kw)
        self.cfg = cfg
        self.aux_loss = None
        if cfg.activation == "swiglu":
            assert cfg.input_dim == cfg.output_dim
            cap = 0.0
            self.moe = SERMoE(cfg.input_dim, cfg.hidden_dim, cfg.num_experts, cfg.top_k, capacity_factor=cap,
                              aux_loss_coef=cfg.load_balance_coef, z_loss_coef=cfg.z_loss_coef, dtype=dtype, device=device)
            return
        self.moe = None
        E, i, h, o = cfg.num_experts, cfg.input_dim, cfg.hidden_dim, cfg.output_dim
        self.router = Linear(i, E, bias=True, dtype=dtype, device=device)
        mk = lambda *s, std: tnn.Parameter(torch.randn(*s, dtype=dtype, device=device) * std)  # noqa: E731
        self.w1, self.b1 = mk(E, h, i, std=1 / math.sqrt(i)), tnn.Parameter(torch.zeros(E, h, dtype=dtype, device=device))
        self.w2, self.b2 = mk(E, o, h, std=1 / math.sqrt(h)), tnn.Parameter(torch.zeros(E, o, dtype=dtype, device=device))

    def forward(self, x):
        if self.moe is not None:
            y = self.moe(x)
            self.aux_loss = self.moe.aux_loss
            return y
        cfg = self.cfg
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        logits = self.router(x2).float()
        idx, w, probs, counts = SERRoute.topk_gating(logits, cfg.top_k, cfg.noisy_gating and self.training, cfg.temperature)
        self.aux_loss = cfg.load_balance_coef * SERRoute.load_balance_loss(probs, counts, cfg.top_k) + \
            cfg.z_loss_coef * SERLoss.z_loss(logits)
        if cfg.enforce_capacity:
            cap = cfg.capacity or max(1, (cfg.input_dim * 2) // cfg.num_experts)
            idx, w = SERRoute.enforce_capacity(idx, w, cfg.num_experts, cap)
        act = _ACT[cfg.activation]
        y = x2.new_zeros(x2.shape[0], cfg.output_dim)
        for e in range(cfg.num_experts):
            tok, slot = (idx == e).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            hdn = act(ops.linear(x2[tok], self.w1[e], self.b1[e]))
            out = ops.linear(hdn, self.w2[e], self.b2[e])
            y.index_add_(0, tok, (out.float() * w[tok, slot].unsqueeze(-1)).to(y.dtype))
        return y.view(*shape[:-1], cfg.output_dim)


class SERModel(Module):
    def __init__(self, cfg: SERConfig = None, dtype=None, device=None, **kw):
        super().__init__()
        cfg = cfg or SERConfig(**kw)
        self.cfg = cfg
        self.layers = tnn.ModuleList([SERLayer(cfg, dtype=dtype, device=device) for _ in range(cfg.num_layers)])

    def forward(self, x):
        from ..utils.observability import bench_marker
        aux = 0.0
        for layer in self.layers:
            bench_marker("SER layer forward start")
            x = layer(x)
            bench_marker("SER layer forward done")
            aux = aux + layer.aux_loss
        self.aux_loss = aux
        return x

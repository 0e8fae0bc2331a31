"""SER (sparse expert routing) layer: softmax router -> top-k -> gated experts (+ shared experts) with the
reference's auxiliary losses. Defaults follow ``SNEPPX_ser_layer`` (E=8, k=2, coef 0.01;
algorithms/ser/core/expert.c:30-39); experts here are gated (SwiGLU) FFNs held as two stacked weight tensors so
that all experts of a rank run as two grouped GEMMs."""
from __future__ import annotations

import math

import torch
import torch.nn as tnn

from ..ops import functional as ops
from ..ops import moe as moe_ops
from .modules import Linear, Module, SwiGLU


class SERMoE(Module):
    def __init__(self, d_model, d_ff, num_experts=8, top_k=2, num_shared_experts=0, capacity_factor=0.0,
                 aux_loss_coef=0.01, z_loss_coef=0.0, act="silu", renorm=True, dtype=None, device=None,
                 init_std=0.02, ep_group=None, expert_fp8=False):
        super().__init__()
        self.d_model, self.d_ff, self.E, self.k = d_model, d_ff, num_experts, top_k
        self.capacity_factor, self.aux_coef, self.z_coef = capacity_factor, aux_loss_coef, z_loss_coef
        self.act, self.renorm = act, renorm
        # forward expert GEMMs in block-scaled fp8 (e4m3 data, 1 x 128 activation / 128 x 128 weight scales)
        self.expert_fp8 = expert_fp8 and d_model % 128 == 0 and d_ff % 128 == 0
        self.router = Linear(d_model, num_experts, bias=False, dtype=dtype, device=device, init_std=init_std)
        self.ep_group = ep_group
        self.ep_world = 1
        self.ep_rank = 0
        if ep_group is not None:
            import torch.distributed as dist
            self.ep_world, self.ep_rank = dist.get_world_size(ep_group), dist.get_rank(ep_group)
        assert num_experts % self.ep_world == 0
        self.E_local = num_experts // self.ep_world
        self.w1 = tnn.Parameter(torch.empty(self.E_local, 2 * d_ff, d_model, dtype=dtype, device=device))
        self.w2 = tnn.Parameter(torch.empty(self.E_local, d_model, d_ff, dtype=dtype, device=device))
        tnn.init.normal_(self.w1, std=init_std)
        tnn.init.normal_(self.w2, std=init_std)
        self.w1.is_expert = self.w2.is_expert = True
        self.shared = SwiGLU(d_model, d_ff * num_shared_experts, act, dtype=dtype, device=device,
                             init_std=init_std) if num_shared_experts else None
        self.aux_loss = None
        self.last_counts = None
        self._ep = None

    def forward(self, x):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        T = x2.shape[0]
        logits = ops.linear(x2, self.router.weight).float()
        idx, w, probs, counts = moe_ops.route(logits, self.k, self.renorm)
        lb, z = moe_ops.aux_losses(logits, probs, counts, self.k)
        self.aux_loss = self.aux_coef * lb + self.z_coef * z
        self.last_counts = counts
        if self.capacity_factor and self.capacity_factor > 0:
            cap = int(math.ceil(self.capacity_factor * T * self.k / self.E))
            idx, w = moe_ops.enforce_capacity(idx, w, self.E, cap)
        if self.ep_world > 1:
            from ..parallel.expert import ep_experts_forward, ep_plan
            plan = ep_plan(self, x2, idx)        # plan kernels first; the shared experts run while the host reads its size
            base = self.shared(x2) if self.shared is not None else None
            y = ep_experts_forward(self, x2, idx, w, base, plan=plan)
            return y.view(shape)
        base = self.shared(x2) if self.shared is not None else None
        no_cap = not (self.capacity_factor and self.capacity_factor > 0)      # nothing was dropped: no need to look
        y = moe_ops.experts_forward(x2, idx, w, self.w1, self.w2, base, self.act, fp8=self.expert_fp8,
                                    all_valid=True if no_cap else None)
        return y.view(shape)

"""Training engine for tensor-parallel x data-parallel models (``TPMamba2ForCausalLM``): ranks are laid out as
``dp`` groups of ``tp`` consecutive ranks. Per step: forward / backward on the TP-sharded model, one all-reduce of the
replicated parameters' gradients over the TP group (they saw only this rank's token rows), one all-reduce of the whole
flat gradient over the DP group, a global gradient norm that counts sharded parameters once per shard and replicated
parameters once, and the fused AdamW step on flat fp32 master weights.

The reference has the sizes in its distributed config (``tensor_parallel_size``, data parallel = world / tp,
include/neural_core/architecture/distributed.h:45-50) and no code that combines them.
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.distributed as dist

from ..optim.fused import adamw_flat_
from ..training.engine import FlatParams


def make_tp_dp_groups(tp: int) -> Tuple[object, object, int, int]:
    """(tp_group, dp_group, tp_rank, dp_rank) for this rank; every rank must call it (groups are created collectively)."""
    world, rank = dist.get_world_size(), dist.get_rank()
    assert world % tp == 0, "world size must be a multiple of the tensor-parallel size"
    dp = world // tp
    tp_group = dp_group = None
    for i in range(dp):
        g = dist.new_group(list(range(i * tp, (i + 1) * tp)))
        if rank // tp == i:
            tp_group = g
    for j in range(tp):
        g = dist.new_group(list(range(j, world, tp)))
        if rank % tp == j:
            dp_group = g
    return tp_group, dp_group, rank % tp, rank // tp


class TPDPEngine:
    def __init__(self, model, tp_group, dp_group, lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, max_grad_norm=1.0):
        self.model, self.tp_group, self.dp_group = model, tp_group, dp_group
        self.dp = dist.get_world_size(dp_group)
        rep = model.replicated_parameters()
        rep_ids = {id(p) for p in rep}
        seen, sharded = set(), []
        for p in model.parameters():
            if p.requires_grad and id(p) not in rep_ids and id(p) not in seen:
                seen.add(id(p))
                sharded.append(p)
        # replicated parameters first: their gradients form one contiguous range for the TP all-reduce
        self.fp = FlatParams(model, params=list(rep) + sharded)
        self.rep_end = self.fp.offsets[len(rep)] if sharded else self.fp.total
        self.master = self.fp.flat.float()
        self.m, self.v = torch.zeros_like(self.master), torch.zeros_like(self.master)
        self.lr, self.betas, self.eps, self.wd, self.max_grad_norm = lr, betas, eps, weight_decay, max_grad_norm
        self.step_count, self.last_norm = 0, None

    def step(self, input_ids, labels):
        """One optimizer step on this DP replica's batch. Returns the mean loss of this replica's batch (summed over
        its TP ranks), as a detached device scalar."""
        self.fp.begin_step()
        loss = self.model(input_ids, labels=labels)["loss"]
        loss.backward()
        self.fp.finalize_grads()
        g = self.fp.grad
        dist.all_reduce(g[: self.rep_end], group=self.tp_group)
        if self.dp > 1:
            g.div_(self.dp)
            dist.all_reduce(g, group=self.dp_group)
        gf = g.float()
        ss_sharded = gf[self.rep_end:].pow(2).sum()
        dist.all_reduce(ss_sharded, group=self.tp_group)
        norm = (gf[: self.rep_end].pow(2).sum() + ss_sharded).sqrt()
        self.last_norm = norm
        clip = torch.clamp(self.max_grad_norm / (norm + 1e-6), max=1.0).reshape(1).float() if self.max_grad_norm > 0 else None
        self.step_count += 1
        p16 = self.fp.flat if self.fp.flat.dtype != torch.float32 else None
        adamw_flat_(self.master if p16 is not None else self.fp.flat, self.m, self.v, g, p16, self.lr, self.betas[0], self.betas[1],
                    self.eps, self.wd, self.step_count, 1.0, clip)
        if p16 is None:
            self.master = self.fp.flat
        total = loss.detach().clone()
        dist.all_reduce(total, group=self.tp_group)
        return total

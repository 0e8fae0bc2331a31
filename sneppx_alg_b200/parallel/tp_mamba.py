"""Tensor-parallel Mamba-2 block: heads (and B / C groups) are split over the TP ranks, activations between blocks are
sequence-parallel (each rank holds T / tp token rows).

    u_s [T/tp, d] --all-gather -> GEMM (in_proj, column parallel)--> z, xBC, dt for this rank's heads, all T tokens
      -> causal conv1d + SiLU over the local channels -> SSD scan over the local heads / groups
      -> gate with z -> RMSNorm over the full d_inner (the sum of squares is all-reduced: one float per token)
      -> GEMM -> reduce-scatter (out_proj, row parallel) -> y_s [T/tp, d]

The two GEMMs are the fused all-gather->GEMM / GEMM->reduce-scatter kernels of ``parallel/tp.py`` on GPUs and
``torch.distributed`` collectives around the plain GEMM on CPU ranks. The reference declares ``sneppx_tp_*`` and
``sneppx_mamba2_*`` separately (kernel/distributed/tensor_parallel.c:40-108, kernel/arch/mamba2.c:36-133) and never
combines them; the sharding follows the baseline configuration "in_proj column-parallel, out_proj row-parallel,
RMSNorm-gated output". Requires nheads % tp == 0 and ngroups % tp == 0.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as tnn
import torch.nn.functional as F

from ..nn.modules import Module
from ..nn.ssm import Mamba2Block
from ..ops import ssm
from .tp import ColumnParallelLinear, RowParallelLinear, TPContext


class _AllReduceSum(torch.autograd.Function):
    """y = sum over ranks of x. Every rank's loss depends on y, so dL/dx = sum over ranks of dL/dy: the backward is
    the same all-reduce applied to the gradient."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        y = x.clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        g = g.clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class TPMamba2Block(Module):
    def __init__(self, d_model, tp: TPContext, d_state=128, d_conv=4, expand=2, headdim=64, ngroups=1, chunk_size=256,
                 eps=1e-5, dtype=None, device=None, init_std=0.02):
        super().__init__()
        w = tp.world
        self.tp, self.d_model, self.d_state, self.d_conv, self.headdim, self.chunk, self.eps = \
            tp, d_model, d_state, d_conv, headdim, chunk_size, eps
        self.d_inner = expand * d_model
        nheads = self.d_inner // headdim
        assert nheads % w == 0 and ngroups % w == 0, "heads and groups must divide over the tensor-parallel ranks"
        self.h_l, self.g_l, self.di_l = nheads // w, ngroups // w, self.d_inner // w
        self.conv_dim_l = self.di_l + 2 * self.g_l * d_state
        cols_l = 2 * self.di_l + 2 * self.g_l * d_state + self.h_l
        self.in_proj = ColumnParallelLinear(d_model, cols_l * w, tp, dtype=dtype, device=device, init_std=init_std)
        self.conv_weight = tnn.Parameter(torch.zeros(self.conv_dim_l, d_conv, dtype=dtype, device=device))
        self.conv_bias = tnn.Parameter(torch.zeros(self.conv_dim_l, dtype=dtype, device=device))
        self.dt_bias = tnn.Parameter(torch.zeros(self.h_l, device=device, dtype=torch.float32))
        self.A_log = tnn.Parameter(torch.zeros(self.h_l, device=device, dtype=torch.float32))
        self.D = tnn.Parameter(torch.ones(self.h_l, device=device, dtype=torch.float32))
        self.norm_weight = tnn.Parameter(torch.ones(self.di_l, dtype=dtype, device=device))
        self.out_proj = RowParallelLinear(self.d_inner, d_model, tp, dtype=dtype, device=device, init_std=init_std)

    @classmethod
    def from_full(cls, full: Mamba2Block, tp: TPContext):
        """This rank's shard of an unsharded block (same parameters, sliced by head / group)."""
        p = full.in_proj.weight
        blk = cls(full.d_model, tp, full.d_state, full.d_conv, full.d_inner // full.d_model, full.headdim, full.ngroups,
                  full.chunk, full.norm.eps, dtype=p.dtype, device=p.device)
        r, di, gn = tp.rank, full.d_inner, full.ngroups * full.d_state
        di_l, gn_l, h_l = blk.di_l, blk.g_l * full.d_state, blk.h_l
        sl = lambda base, width: slice(base + r * width, base + (r + 1) * width)  # noqa: E731
        rows = [sl(0, di_l), sl(di, di_l), sl(2 * di, gn_l), sl(2 * di + gn, gn_l), sl(2 * di + 2 * gn, h_l)]
        chans = [sl(0, di_l), sl(di, gn_l), sl(di + gn, gn_l)]
        with torch.no_grad():
            blk.in_proj.weight.copy_(torch.cat([full.in_proj.weight[s] for s in rows]))
            blk.conv_weight.copy_(torch.cat([full.conv_weight[s] for s in chans]))
            blk.conv_bias.copy_(torch.cat([full.conv_bias[s] for s in chans]))
            for name in ("dt_bias", "A_log", "D"):
                getattr(blk, name).copy_(getattr(full, name)[sl(0, h_l)])
            blk.norm_weight.copy_(full.norm.weight[sl(0, di_l)])
            blk.out_proj.weight.copy_(full.out_proj.weight[:, sl(0, di_l)])
        return blk

    def forward(self, u_s, batch: int, residual=None):
        """u_s [T/tp, d_model]: this rank's rows of the flattened [batch * L, d_model] activations (rank r holds rows
        r * T/tp ..). Returns y_s [T/tp, d_model] (+ residual)."""
        N, P = self.d_state, self.headdim
        zxbcdt = self.in_proj(u_s)                                   # [T, local columns]
        T = zxbcdt.shape[0]
        L = T // batch
        z, xBC, dt = torch.split(zxbcdt, [self.di_l, self.conv_dim_l, self.h_l], dim=-1)
        xBC = ssm.causal_conv1d(xBC.reshape(batch, L, self.conv_dim_l), self.conv_weight, self.conv_bias, act=True)
        x, Bm, Cm = torch.split(xBC, [self.di_l, self.g_l * N, self.g_l * N], dim=-1)
        dt = F.softplus(dt.float().reshape(batch, L, self.h_l) + self.dt_bias)
        y = ssm.ssd_scan(x.reshape(batch, L, self.h_l, P), dt, -torch.exp(self.A_log), Bm.reshape(batch, L, self.g_l, N),
                         Cm.reshape(batch, L, self.g_l, N), self.D, chunk=min(self.chunk, 128))
        y = ssm.gate_mul(y.reshape(batch, L, self.di_l), z.reshape(batch, L, self.di_l))
        # RMSNorm over the full d_inner: local sums of squares, one all-reduced float per token
        yf = y.float()
        total = _AllReduceSum.apply(yf.pow(2).sum(-1, keepdim=True), self.tp.group)
        yn = (yf * torch.rsqrt(total / self.d_inner + self.eps) * self.norm_weight.float()).to(y.dtype)
        return self.out_proj(yn.reshape(T, self.di_l), residual=residual)


class TPMamba2ForCausalLM(Module):
    """Mamba-2 language model with tensor-parallel mixers and sequence-parallel activations. Embedding, norms and the
    tied LM head are replicated and act on this rank's token rows only, so their gradients are partial sums over
    tokens: call ``sync_replicated_grads`` after backward (before the optimizer or the data-parallel reduction)."""

    def __init__(self, full_model, tp: TPContext):
        """Shards an unsharded ``Mamba2ForCausalLM`` (every rank passes the same model, e.g. built from one seed)."""
        super().__init__()
        self.config, self.tp = full_model.config, tp
        self.embedding, self.norm, self.lm_head = full_model.embedding, full_model.norm, full_model.lm_head
        self.layer_norms = tnn.ModuleList([l.norm for l in full_model.layers])
        self.mixers = tnn.ModuleList([TPMamba2Block.from_full(l.mixer, tp) for l in full_model.layers])

    def head_weight(self):
        return self.embedding.weight if self.lm_head is None else self.lm_head.weight

    def replicated_parameters(self):
        return [p for p in self.parameters() if getattr(p, "tensor_parallel", None) is None and not any(
            p is q for m in self.mixers for q in (m.conv_weight, m.conv_bias, m.dt_bias, m.A_log, m.D, m.norm_weight))]

    def sync_replicated_grads(self):
        for p in self.replicated_parameters():
            if p.grad is not None:
                dist.all_reduce(p.grad, group=self.tp.group)

    def forward(self, input_ids, labels=None):
        """input_ids, labels [B, L] (the same on every TP rank). Returns this rank's share of the summed token loss
        divided by the global number of target tokens, so that the sum over TP ranks is the mean loss."""
        from ..ops import functional as ops
        B, L = input_ids.shape
        T, w, r = B * L, self.tp.world, self.tp.rank
        rows = slice(r * T // w, (r + 1) * T // w)
        delta, resid = self.embedding(input_ids.reshape(T)[rows]), None
        for norm, mixer in zip(self.layer_norms, self.mixers):
            if resid is None:
                h, resid = norm(delta), delta
            else:
                h, resid = norm(delta, residual=resid)
            delta = mixer(h, batch=B)
        h, _ = self.norm(delta, residual=resid)
        if labels is None:
            return {"hidden_rows": h}
        tgt = torch.full_like(labels, -100)
        tgt[:, :-1] = labels[:, 1:]
        tgt_rows = tgt.reshape(T)[rows]
        n_local, n_total = int((tgt_rows != -100).sum()), int((tgt != -100).sum())
        loss = ops.linear_cross_entropy(h, self.head_weight(), tgt_rows) if n_local else h.sum() * 0
        return {"loss": loss * (n_local / max(n_total, 1))}

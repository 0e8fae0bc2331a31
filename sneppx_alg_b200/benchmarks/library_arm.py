"""Library comparator for the training benchmarks: the same three model shapes and the same step, stated with
PyTorch library ops only and NCCL collectives from ``torch.distributed``. Nothing in this file imports this
package's kernels, ops or engines; it is what a PyTorch user gets on the same box without them.

* models: ``LibLlama`` (dense GQA decoder), ``LibDeepSeek`` (MHA + SER MoE with expert parallelism through
  ``all_to_all_single``), ``LibMamba2`` (chunked SSD as batched matmuls, tensor parallel through all-gather /
  reduce-scatter). cuBLAS through ``F.linear`` / ``einsum``, ``scaled_dot_product_attention``, ``F.rms_norm``,
  ``F.conv1d``, ``F.cross_entropy``.
* ``LibZeroEngine``: bucketed flat bf16 parameters and gradients, fp32 master weights and moments on each rank's
  shard, torch's fused AdamW, global-norm clipping. Communication is overlapped the way stock FSDP does it:
  a bucket's gradient reduce-scatter is issued on a side stream as soon as backward has produced the bucket,
  and the updated parameters are all-gathered bucket by bucket on the side stream, each layer waiting only for
  its own bucket.

The reference states the intended behaviour (gather -> forward -> free, reduce-scatter of gradients:
interface_bindings/fsdp.py:78-247; expert all-to-all: kernel/distributed/expert_parallel.c:70-116; column /
row parallel linears: kernel/distributed/tensor_parallel.c:40-108) but its collectives are local copies.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


def _rope_tables(S, D, theta, device):
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, device=device, dtype=torch.float32) / D))
    ang = torch.outer(torch.arange(S, device=device, dtype=torch.float32), inv)
    return ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]


def _rope(x, cos, sin):
    D = x.shape[-1]
    x1, x2 = x[..., : D // 2].float(), x[..., D // 2:].float()
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), -1).to(x.dtype)


def _param(*shape, std=0.02, dtype=None, device=None, ones=False):
    p = nn.Parameter(torch.empty(*shape, dtype=dtype, device=device))
    with torch.no_grad():
        p.fill_(1.0) if ones else p.normal_(0.0, std)
    return p


class _Attention(nn.Module):
    def __init__(self, d, H, Hk, D, dtype, device):
        super().__init__()
        self.H, self.Hk, self.D = H, Hk, D
        self.qkv = _param((H + 2 * Hk) * D, d, dtype=dtype, device=device)
        self.o = _param(d, H * D, dtype=dtype, device=device)

    def forward(self, h, cos, sin):
        B, S, _ = h.shape
        H, Hk, D = self.H, self.Hk, self.D
        qkv = F.linear(h, self.qkv)
        q = _rope(qkv[..., : H * D].view(B, S, H, D), cos, sin).transpose(1, 2)
        k = _rope(qkv[..., H * D:(H + Hk) * D].view(B, S, Hk, D), cos, sin).transpose(1, 2)
        v = qkv[..., (H + Hk) * D:].view(B, S, Hk, D).transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=H != Hk)
        return F.linear(a.transpose(1, 2).reshape(B, S, H * D), self.o)


class _SwiGLU(nn.Module):
    def __init__(self, d, ff, dtype, device):
        super().__init__()
        self.gu = _param(2 * ff, d, dtype=dtype, device=device)
        self.down = _param(d, ff, dtype=dtype, device=device)

    def forward(self, h):
        g, u = F.linear(h, self.gu).chunk(2, -1)
        return F.linear(F.silu(g) * u, self.down)


class _DecoderLayer(nn.Module):
    def __init__(self, cfg, mlp, dtype, device):
        super().__init__()
        d = cfg.hidden_size
        self.eps = cfg.rms_norm_eps
        self.n1 = _param(d, ones=True, dtype=dtype, device=device)
        self.n2 = _param(d, ones=True, dtype=dtype, device=device)
        self.attn = _Attention(d, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, dtype, device)
        self.mlp = mlp

    def forward(self, x, cos, sin):
        d = x.shape[-1]
        x = x + self.attn(F.rms_norm(x, (d,), self.n1, self.eps), cos, sin)
        return x + self.mlp(F.rms_norm(x, (d,), self.n2, self.eps))


class _LM(nn.Module):
    """Embedding, a ModuleList of layers, final norm, (tied) head and the shifted cross-entropy."""

    def _init_lm(self, cfg, dtype, device, vocab=None):
        self.cfg = cfg
        self.V = vocab or cfg.vocab_size
        self.emb = _param(self.V, cfg.hidden_size, dtype=dtype, device=device)
        self.nf = _param(cfg.hidden_size, ones=True, dtype=dtype, device=device)
        self.head = None if cfg.tie_word_embeddings else _param(self.V, cfg.hidden_size, dtype=dtype, device=device)

    def _loss(self, x, ids):
        x = F.rms_norm(x, (x.shape[-1],), self.nf, self.cfg.rms_norm_eps)
        logits = F.linear(x[:, :-1], self.emb if self.head is None else self.head)
        return F.cross_entropy(logits.reshape(-1, self.V).float(), ids[:, 1:].reshape(-1))


class LibLlama(_LM):
    def __init__(self, cfg, dtype=torch.bfloat16, device=None, layers=0):
        super().__init__()
        self._init_lm(cfg, dtype, device)
        self.layers = nn.ModuleList([_DecoderLayer(cfg, _SwiGLU(cfg.hidden_size, cfg.intermediate_size, dtype, device),
                                                   dtype, device) for _ in range(layers or cfg.num_hidden_layers)])

    def forward(self, ids):
        cos, sin = _rope_tables(ids.shape[1], self.cfg.head_dim, self.cfg.rope_theta, ids.device)
        x = F.embedding(ids, self.emb)
        for layer in self.layers:
            x = layer(x, cos, sin)
        return self._loss(x, ids)


# ------------------------------------------------------------------------------ SER MoE, expert parallel
def _a2a(x, out_splits, in_splits, group):
    """Differentiable all_to_all_single along dim 0 (identity without a group)."""
    if group is None:
        return x
    import torch.distributed.nn.functional as dfn
    out = torch.empty(sum(out_splits), *x.shape[1:], dtype=x.dtype, device=x.device)
    return dfn.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)


class _MoE(nn.Module):
    """Softmax router, top-k with renormalised weights, load-balance loss E * sum_e f_e p_e (/k), routed SwiGLU
    experts split contiguously over the EP ranks, shared experts on every rank. No token is dropped: the
    all-to-all carries exactly the routed rows (split sizes are read back to the host, as NCCL needs them)."""

    grouped_mm = True       # use torch._grouped_mm for the expert projections while it works on this device

    def __init__(self, cfg, dtype, device, ep_group=None):
        super().__init__()
        d, ff = cfg.hidden_size, cfg.moe_intermediate_size
        self.E, self.k, self.coef = cfg.num_experts, cfg.num_experts_per_token, cfg.router_aux_loss_coef
        self.group = ep_group
        self.world = dist.get_world_size(ep_group) if ep_group is not None else 1
        self.E_local = self.E // self.world
        self.router = _param(self.E, d, dtype=dtype, device=device)
        self.w1 = _param(self.E_local, 2 * ff, d, dtype=dtype, device=device)
        self.w2 = _param(self.E_local, d, ff, dtype=dtype, device=device)
        self.w1.is_expert = self.w2.is_expert = True
        self.shared = _SwiGLU(d, ff * cfg.num_shared_experts, dtype, device) if cfg.num_shared_experts else None
        self.aux = None

    def forward(self, h):
        shape = h.shape
        x = h.reshape(-1, shape[-1])
        T, d = x.shape
        E, k, w_, El = self.E, self.k, self.world, self.E_local
        probs = torch.softmax(F.linear(x, self.router).float(), -1)
        w, idx = probs.topk(k, dim=-1)
        w = w / w.sum(-1, keepdim=True)
        flat_e = idx.reshape(-1)
        counts = torch.bincount(flat_e, minlength=E)
        self.aux = self.coef * E * ((counts.float() / T).detach() * probs.mean(0)).sum() / k
        order = torch.argsort(flat_e, stable=True)            # by expert, hence by owner rank
        tok = order // k
        send_ce = counts.view(w_, El)
        if self.group is not None:
            recv_ce = torch.empty_like(send_ce)
            dist.all_to_all_single(recv_ce, send_ce.contiguous(), group=self.group)
        else:
            recv_ce = send_ce
        sc, rc = send_ce.sum(1).tolist(), recv_ce.sum(1).tolist()
        recv_x = _a2a(x[tok], rc, sc, self.group)
        # received rows come ordered by (source rank, local expert): regroup them by expert
        eid = torch.arange(El, device=x.device).repeat(w_).repeat_interleave(recv_ce.reshape(-1), output_size=sum(rc))
        perm = torch.argsort(eid, stable=True)
        xs = recv_x[perm]
        per_expert = recv_ce.sum(0)
        ys_sorted = None
        if _MoE.grouped_mm and hasattr(torch, "_grouped_mm"):
            # one grouped GEMM per projection over the expert-sorted rows (row offsets stay on the device)
            try:
                offs = per_expert.cumsum(0).to(torch.int32)
                g, u = torch._grouped_mm(xs, self.w1.transpose(1, 2), offs=offs).chunk(2, -1)
                ys_sorted = torch._grouped_mm(F.silu(g) * u, self.w2.transpose(1, 2), offs=offs)
            except (RuntimeError, NotImplementedError):
                _MoE.grouped_mm = False        # this build / device has no grouped GEMM: loop over the experts
        if ys_sorted is None:
            outs = []
            for chunk, w1e, w2e in zip(xs.split(per_expert.tolist()), self.w1.unbind(0), self.w2.unbind(0)):
                if chunk.shape[0] == 0:
                    outs.append(chunk)
                    continue
                g, u = F.linear(chunk, w1e).chunk(2, -1)
                outs.append(F.linear(F.silu(g) * u, w2e))
            ys_sorted = torch.cat(outs)
        ys = torch.empty_like(xs).index_copy(0, perm, ys_sorted)
        back = _a2a(ys, sc, rc, self.group)
        y = torch.zeros(T, d, dtype=torch.float32, device=x.device).index_add(
            0, tok, back.float() * w.reshape(-1)[order].unsqueeze(1))
        if self.shared is not None:
            y = y + self.shared(x).float()
        return y.to(h.dtype).view(shape)


class LibDeepSeek(_LM):
    """DeepSeek-V2-Lite shape with plain multi-head attention: dense SwiGLU in the first layer(s), SER MoE after."""

    def __init__(self, cfg, dtype=torch.bfloat16, device=None, ep_group=None, layers=0):
        super().__init__()
        self._init_lm(cfg, dtype, device)
        n = layers or cfg.num_hidden_layers
        self.layers = nn.ModuleList([
            _DecoderLayer(cfg, _SwiGLU(cfg.hidden_size, cfg.intermediate_size, dtype, device)
                          if i < cfg.first_dense_layers else _MoE(cfg, dtype, device, ep_group), dtype, device)
            for i in range(n)])

    def forward(self, ids):
        cos, sin = _rope_tables(ids.shape[1], self.cfg.head_dim, self.cfg.rope_theta, ids.device)
        x = F.embedding(ids, self.emb)
        for layer in self.layers:
            x = layer(x, cos, sin)
        loss = self._loss(x, ids)
        for layer in self.layers:
            if isinstance(layer.mlp, _MoE):
                loss = loss + layer.mlp.aux
        return loss


# ------------------------------------------------------------------------------ Mamba-2, tensor parallel
def _rs_sum(x, group):
    """Sum over ranks, this rank's block of rows (reduce-scatter; all-reduce + slice on back-ends without it)."""
    w, r = dist.get_world_size(group), dist.get_rank(group)
    n = x.shape[0] // w
    if dist.get_backend(group) == "nccl":
        out = torch.empty(n, *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
        return out
    y = x.clone()
    dist.all_reduce(y, group=group)
    return y[r * n:(r + 1) * n].clone()


def _ag(x, group):
    w = dist.get_world_size(group)
    out = torch.empty(w * x.shape[0], *x.shape[1:], dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out


class _AllGatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _ag(x, group)

    @staticmethod
    def backward(ctx, g):
        return _rs_sum(g, ctx.group), None


class _ReduceScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _rs_sum(x, group)

    @staticmethod
    def backward(ctx, g):
        return _ag(g, ctx.group), None


class _AllReduce(torch.autograd.Function):
    """Sum over ranks in forward and in backward (every rank's loss depends on the sum)."""

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


class _GradAllReduce(torch.autograd.Function):
    """Identity in forward; the gradient is summed over the ranks (parameters replicated over tensor-parallel
    ranks that each see only part of the tokens)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


def _rep(p, group):
    return p if group is None else _GradAllReduce.apply(p, group)


def ssd_chunked(x, dt, A, Bm, Cm, D, chunk):
    """Mamba-2 SSD as batched matmuls. x [B,L,H,P], dt [B,L,H] (> 0), A [H] (< 0), Bm / Cm [B,L,G,N], D [H].
    h_t = exp(dt_t A) h_{t-1} + dt_t B_t x_t^T,  y_t = C_t h_t + D x_t, evaluated chunk by chunk: a masked
    (C B^T * decay) x product inside each chunk, one state per chunk, and a chunk-level recurrence between them."""
    Bsz, L, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    Q = min(chunk, L)
    assert L % Q == 0
    C_ = L // Q
    rep = H // G
    dA = (dt.float() * A.float()).view(Bsz, C_, Q, H)
    cum = dA.cumsum(2)                                                   # [B,C,Q,H]
    xb = (x.float() * dt.float().unsqueeze(-1)).to(x.dtype).view(Bsz, C_, Q, G, rep, P)
    Bc, Cc = Bm.view(Bsz, C_, Q, G, N), Cm.view(Bsz, C_, Q, G, N)
    # inside a chunk
    cb = torch.einsum("bcign,bcjgn->bcgij", Cc, Bc)                      # [B,C,G,Q,Q]
    ch = cum.permute(0, 1, 3, 2)                                         # [B,C,H,Q]
    seg = ch.unsqueeze(-1) - ch.unsqueeze(-2)                            # cum_i - cum_j
    mask = torch.ones(Q, Q, dtype=torch.bool, device=x.device).tril()
    decay = torch.exp(seg.masked_fill(~mask, float("-inf"))).view(Bsz, C_, G, rep, Q, Q)
    m = (cb.unsqueeze(3).float() * decay).to(x.dtype)                    # [B,C,G,rep,Q,Q]
    y = torch.einsum("bcgrij,bcjgrp->bcigrp", m, xb)
    # one state per chunk: sum_j exp(cum_last - cum_j) B_j xbar_j^T
    to_end = torch.exp(cum[:, :, -1:, :] - cum).view(Bsz, C_, Q, G, rep)
    states = torch.einsum("bcjgn,bcjgrp->bcgrpn", Bc, (xb.float() * to_end.unsqueeze(-1)).to(x.dtype)).float()
    # recurrence over chunks: state entering chunk c
    tot = cum[:, :, -1, :].view(Bsz, C_, G, rep)                         # log-decay of a whole chunk
    tc = torch.cat([torch.zeros_like(tot[:, :1]), tot], 1).cumsum(1)     # [B,C+1,...]
    segc = tc[:, :-1].unsqueeze(2) - tc[:, 1:].unsqueeze(1)              # [B, c (target), c' (source), G, rep]
    maskc = torch.ones(C_, C_, dtype=torch.bool, device=x.device).tril(-1)
    dec_c = torch.exp(segc.masked_fill(~maskc.view(1, C_, C_, 1, 1), float("-inf")))
    enter = torch.einsum("bzcgr,bcgrpn->bzgrpn", dec_c, states)          # [B,C,G,rep,P,N]
    y = y + torch.einsum("bcign,bcgrpn->bcigrp", Cc, enter.to(x.dtype)) * \
        torch.exp(cum).view(Bsz, C_, Q, G, rep, 1).to(x.dtype)
    y = y.reshape(Bsz, L, H, P)
    return y + x * D.to(x.dtype).view(1, 1, H, 1)


class _Mamba2Mixer(nn.Module):
    def __init__(self, cfg, dtype, device, tp_group=None):
        super().__init__()
        d, N, P = cfg.hidden_size, cfg.ssm_state_size, cfg.ssm_head_dim
        self.group = tp_group
        w = dist.get_world_size(tp_group) if tp_group is not None else 1
        self.d_inner = cfg.ssm_expand * d
        self.h_l, self.g_l, self.di_l = self.d_inner // P // w, cfg.ssm_ngroups // w, self.d_inner // w
        self.N, self.P, self.K, self.chunk, self.eps = N, P, cfg.ssm_conv_kernel, cfg.ssm_chunk_size, cfg.rms_norm_eps
        self.conv_dim = self.di_l + 2 * self.g_l * N
        self.in_proj = _param(2 * self.di_l + 2 * self.g_l * N + self.h_l, d, dtype=dtype, device=device)
        self.conv_w = _param(self.conv_dim, 1, self.K, std=0.2, dtype=dtype, device=device)
        self.conv_b = nn.Parameter(torch.zeros(self.conv_dim, dtype=dtype, device=device))
        dtv = torch.exp(torch.rand(self.h_l, device=device) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
        self.dt_bias = nn.Parameter(dtv + torch.log(-torch.expm1(-dtv)))          # softplus(dt_bias) in [1e-3, 1e-1]
        self.A_log = nn.Parameter(torch.log(torch.empty(self.h_l, device=device).uniform_(1, 16)))
        self.D = nn.Parameter(torch.ones(self.h_l, device=device))
        self.norm_w = _param(self.di_l, ones=True, dtype=dtype, device=device)
        self.out_proj = _param(d, self.di_l, dtype=dtype, device=device)

    def forward(self, u, batch):
        """u [T_local, d] (this rank's token rows when tensor parallel) -> [T_local, d]."""
        if self.group is not None:
            u = _AllGatherRows.apply(u, self.group)
        T = u.shape[0]
        L = T // batch
        z, xBC, dt = F.linear(u, self.in_proj).split([self.di_l, self.conv_dim, self.h_l], -1)
        xBC = xBC.reshape(batch, L, self.conv_dim).transpose(1, 2)
        xBC = F.silu(F.conv1d(xBC, self.conv_w, self.conv_b, padding=self.K - 1, groups=self.conv_dim)[..., :L])
        xBC = xBC.transpose(1, 2)
        x, Bm, Cm = xBC.split([self.di_l, self.g_l * self.N, self.g_l * self.N], -1)
        dt = F.softplus(dt.float().reshape(batch, L, self.h_l) + self.dt_bias)
        y = ssd_chunked(x.reshape(batch, L, self.h_l, self.P), dt, -torch.exp(self.A_log),
                        Bm.reshape(batch, L, self.g_l, self.N), Cm.reshape(batch, L, self.g_l, self.N), self.D, self.chunk)
        y = (y.reshape(T, self.di_l) * F.silu(z)).float()
        ss = y.pow(2).sum(-1, keepdim=True)
        if self.group is not None:
            ss = _AllReduce.apply(ss, self.group)
        y = (y * torch.rsqrt(ss / self.d_inner + self.eps) * self.norm_w.float()).to(u.dtype)
        out = F.linear(y, self.out_proj)
        return _ReduceScatterRows.apply(out, self.group) if self.group is not None else out


class _Mamba2Layer(nn.Module):
    def __init__(self, cfg, dtype, device, tp_group):
        super().__init__()
        self.group, self.eps = tp_group, cfg.rms_norm_eps
        self.norm = _param(cfg.hidden_size, ones=True, dtype=dtype, device=device)
        self.mixer = _Mamba2Mixer(cfg, dtype, device, tp_group)

    def forward(self, x, batch):
        return x + self.mixer(F.rms_norm(x, (x.shape[-1],), _rep(self.norm, self.group), self.eps), batch)


class LibMamba2(_LM):
    """Mamba-2 language model; with ``tp_group`` the mixers are split by heads / groups over the tensor-parallel
    ranks and the activations between blocks are sequence parallel (each rank keeps T / tp token rows)."""

    def __init__(self, cfg, dtype=torch.bfloat16, device=None, tp_group=None, layers=0):
        super().__init__()
        self._init_lm(cfg, dtype, device, vocab=(cfg.vocab_size + 63) // 64 * 64)
        self.group = tp_group
        self.layers = nn.ModuleList([_Mamba2Layer(cfg, dtype, device, tp_group)
                                     for _ in range(layers or cfg.num_hidden_layers)])

    def forward(self, ids):
        B, L = ids.shape
        g = self.group
        tgt = torch.full_like(ids, -100)
        tgt[:, :-1] = ids[:, 1:]
        flat_ids, flat_tgt = ids.reshape(-1), tgt.reshape(-1)
        if g is not None:
            w, r = dist.get_world_size(g), dist.get_rank(g)
            n = flat_ids.numel() // w
            flat_ids, flat_tgt = flat_ids[r * n:(r + 1) * n], flat_tgt[r * n:(r + 1) * n]
        emb = _rep(self.emb, g)
        x = F.embedding(flat_ids, emb)
        for layer in self.layers:
            x = layer(x, B)
        x = F.rms_norm(x, (x.shape[-1],), _rep(self.nf, g), self.cfg.rms_norm_eps)
        logits = F.linear(x, emb if self.head is None else _rep(self.head, g))
        loss = F.cross_entropy(logits.float(), flat_tgt, ignore_index=-100, reduction="sum")
        return loss / (B * (L - 1))       # summed over the tensor-parallel ranks this is the mean loss


# ------------------------------------------------------------------------------ ZeRO data parallelism on NCCL
class LibZeroEngine:
    """Flat-buffer ZeRO step with torch.distributed collectives and torch's fused AdamW.

    ``group``: the data-parallel group the parameters are sharded over (None: one rank, no communication).
    ``tp_group``: tensor-parallel peers, only used to count gradient norms once. Parameters marked
    ``is_expert`` are not reduced (they differ between ranks) and are updated locally; parameters marked
    ``tp_replicated`` go to the last bucket together with everything outside ``model.layers``."""

    CHUNK = 1 << 28

    def __init__(self, model, group=None, tp_group=None, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1,
                 max_grad_norm=1.0):
        self.model, self.group, self.tp_group, self.max_norm = model, group, tp_group, max_grad_norm
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        params = [p for p in model.parameters() if p.requires_grad]
        dev, dt = params[0].device, params[0].dtype
        self.dev, self.cuda = dev, dev.type == "cuda"
        experts = [p for p in params if getattr(p, "is_expert", False)]
        taken = {id(p) for p in experts}
        buckets: List[List[nn.Parameter]] = []
        self.bucket_modules = []
        for layer in model.layers:
            ps = [p for p in layer.parameters() if id(p) not in taken and not getattr(p, "tp_replicated", False)]
            taken.update(id(p) for p in ps)
            buckets.append(ps)
            self.bucket_modules.append(layer)
        buckets.append([p for p in params if id(p) not in taken])
        self.rest = len(buckets) - 1
        unit = 256 * self.world
        self.bounds, off = [], 0
        slots = []
        for ps in buckets:
            b0 = off
            for p in ps:
                slots.append((p, off))
                off += (p.numel() + 255) // 256 * 256
            off = (off + unit - 1) // unit * unit
            self.bounds.append((b0, off))
        self.flat = torch.zeros(off, dtype=dt, device=dev)
        self.grad = torch.zeros(off, dtype=dt, device=dev)
        self.views = {}
        for p, o in slots:
            v = self.flat[o:o + p.numel()].view_as(p)
            v.copy_(p.data)
            p.data = v
            self.views[id(p)] = self.grad[o:o + p.numel()].view_as(p)
        if self.world > 1:
            dist.broadcast(self.flat, dist.get_global_rank(group, 0), group=group)
        self.shard_off = [b0 // self.world for b0, _ in self.bounds]
        self.shard_total = off // self.world
        self.gshard = torch.zeros(self.shard_total, dtype=dt, device=dev)
        self.pshard = torch.empty(self.shard_total, dtype=dt, device=dev)
        master = torch.empty(self.shard_total, dtype=torch.float32, device=dev)
        for bi, (b0, b1) in enumerate(self.bounds):
            sz = (b1 - b0) // self.world
            master[self.shard_off[bi]: self.shard_off[bi] + sz].copy_(self.flat[b0 + self.rank * sz: b0 + (self.rank + 1) * sz])
        kw = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, fused=True)
        self.master, self.opts = master, []
        for c0 in range(0, self.shard_total, self.CHUNK):
            mp = nn.Parameter(master[c0:c0 + self.CHUNK])
            self.opts.append((c0, mp, torch.optim.AdamW([mp], **kw)))
        # experts: local fp32 master copies, local update
        self.experts = experts
        self.e_master = [nn.Parameter(p.detach().float()) for p in experts]
        self.e_opt = torch.optim.AdamW(self.e_master, **kw) if experts else None
        self.bucket_of, self.pending = {}, []
        for bi, ps in enumerate(buckets):
            self.pending.append(len(ps))
            for p in ps:
                self.bucket_of[id(p)] = bi
                p.register_post_accumulate_grad_hook(self._grad_hook)
        self.comm = torch.cuda.Stream(device=dev) if self.cuda else None
        self.gather_events = [None] * len(buckets)
        for bi, mod in enumerate(self.bucket_modules):
            mod.register_forward_pre_hook(lambda m, a, bi=bi: self._wait_bucket(bi))
        self.last_norm = None

    # -- backward side: copy the finished gradient into the flat buffer; reduce the bucket once it is complete
    def _grad_hook(self, p):
        self.views[id(p)].copy_(p.grad)
        p.grad = None
        bi = self.bucket_of[id(p)]
        self._left[bi] -= 1
        if self._left[bi] == 0 and bi != self.rest:
            self._reduce(bi)

    def _reduce(self, bi):
        b0, b1 = self.bounds[bi]
        sz = (b1 - b0) // self.world
        dst = self.gshard[self.shard_off[bi]: self.shard_off[bi] + sz]
        g = self.grad[b0:b1]
        if self.world == 1:
            dst.copy_(g)
            return
        if self.cuda:
            self.comm.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm):
                dist.reduce_scatter_tensor(dst, g, op=dist.ReduceOp.AVG, group=self.group)
        else:
            gf = g.float()
            dist.all_reduce(gf, group=self.group)
            dst.copy_(gf[self.rank * sz:(self.rank + 1) * sz] / self.world)

    def _wait_bucket(self, bi):
        ev = self.gather_events[bi]
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
            self.gather_events[bi] = None

    def _gather(self, bi):
        b0, b1 = self.bounds[bi]
        sz = (b1 - b0) // self.world
        src = self.pshard[self.shard_off[bi]: self.shard_off[bi] + sz]
        if self.world == 1:
            self.flat[b0:b1].copy_(src)
            return
        if self.cuda:
            with torch.cuda.stream(self.comm):
                dist.all_gather_into_tensor(self.flat[b0:b1], src, group=self.group)
                ev = torch.cuda.Event()
                ev.record(self.comm)
            self.gather_events[bi] = ev
        else:
            dist.all_gather_into_tensor(self.flat[b0:b1], src.contiguous(), group=self.group)

    def step(self, ids):
        self._left = list(self.pending)
        self._wait_bucket(self.rest)
        loss = self.model(ids)
        loss.backward()
        self._reduce(self.rest)
        if self.cuda and self.world > 1:
            torch.cuda.current_stream().wait_stream(self.comm)
        r0 = self.shard_off[self.rest]
        ss = torch.stack([torch.linalg.vector_norm(self.gshard[:r0], dtype=torch.float32).pow(2),
                          torch.linalg.vector_norm(self.gshard[r0:], dtype=torch.float32).pow(2)])
        for p in self.experts:
            ss[0] += torch.linalg.vector_norm(p.grad, dtype=torch.float32).pow(2)
        if self.world > 1:
            dist.all_reduce(ss, group=self.group)
        if self.tp_group is not None:
            dist.all_reduce(ss[0:1], group=self.tp_group)      # sharded parameters: one share per tensor-parallel rank
        nrm = ss.sum().sqrt()
        self.last_norm = nrm
        coef = torch.clamp(self.max_norm / (nrm + 1e-6), max=1.0) if self.max_norm > 0 else torch.ones_like(nrm)
        for c0, mp, opt in self.opts:
            mp.grad = self.gshard[c0:c0 + self.CHUNK].float() * coef
            opt.step()
            mp.grad = None
        self.pshard.copy_(self.master)
        if self.e_opt is not None:
            for p, mp in zip(self.experts, self.e_master):
                mp.grad = p.grad.float() * coef
                p.grad = None
            self.e_opt.step()
            for p, mp in zip(self.experts, self.e_master):
                mp.grad = None
                p.data.copy_(mp.data)
        if self.cuda and self.world > 1:
            self.comm.wait_stream(torch.cuda.current_stream())
        for bi in [self.rest] + list(range(self.rest)):
            self._gather(bi)
        return loss.detach()


def build(model_name, cfg, dev, world, rank, layers=0, tp=1, ep=False):
    """(model, engine, description, data-parallel size, loss_fn) of the library arm for a benchmark config."""
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    arch = getattr(cfg, "architecture", "transformer")
    tp_group = dp_group = None
    dp = world
    if arch == "mamba2":
        if world > 1 and tp > 1:
            dp = world // tp
            for i in range(dp):
                g = dist.new_group(list(range(i * tp, (i + 1) * tp)))
                if rank // tp == i:
                    tp_group = g
            for j in range(tp):
                g = dist.new_group(list(range(j, world, tp)))
                if rank % tp == j:
                    dp_group = g
            if dp == 1:
                dp_group = None
        elif world > 1:
            dp_group = dist.group.WORLD
        model = LibMamba2(cfg, dtype, dev, tp_group, layers)
        if tp_group is not None:
            model.emb.tp_replicated = model.nf.tp_replicated = True
            for layer in model.layers:
                layer.norm.tp_replicated = True
        par = f"tp{tp}xdp{dp} (NCCL all-gather / reduce-scatter, ZeRO-1 over dp)" if tp_group is not None else f"zero-dp{world}"
    elif arch == "deepseek_moe":
        ep_group = dist.group.WORLD if (ep and world > 1) else None
        dp_group = dist.group.WORLD if world > 1 else None
        model = LibDeepSeek(cfg, dtype, dev, ep_group, layers)
        par = f"ep{world}+zero1 (all_to_all_single, no token dropped)" if ep_group is not None else f"zero-dp{world}"
    else:
        dp_group = dist.group.WORLD if world > 1 else None
        model = LibLlama(cfg, dtype, dev, layers)
        par = f"zero-dp{world} (per-layer reduce-scatter in backward and all-gather prefetch on a side stream)"
    engine = LibZeroEngine(model, dp_group, tp_group)
    return model, engine, par, dp, tp_group

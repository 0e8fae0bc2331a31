"""Context (sequence) parallelism: every rank holds S / w tokens of each sequence.

* ``cp_attention``: all-gather-KV attention. K and V of the whole sequence are gathered (differentiable: the backward
  of the gather is a reduce-scatter of dK / dV) and the local queries run through the flash-attention kernel with the
  bottom-right causal alignment (query i sees keys <= i + Skv - Sq), so a rank only reads the keys it can see.
  ``layout="zigzag"`` gives rank r the chunks r and 2w-1-r, which equalises causal work over ranks.
* ``ring_attention``: ring variant with a backward pass (dK / dV accumulators travel with their blocks);
  ``ring_attention_forward``: the inference-only form: K/V blocks travel rank to rank and the per-block outputs
  are merged with their log-sum-exp (no full-sequence K/V is ever resident).
* ``cp_ssd_scan``: Mamba-2 scan over a sharded sequence. Pass 1 scans every shard from a zero state (in parallel) and
  yields the shard's final state and total decay; the [H, P, N] states are all-gathered (a few hundred KB) and each
  rank folds its predecessors' states into its true initial state; pass 2 re-scans with that state. ``mode="serial"``
  instead hands the state rank to rank (one scan per rank, ranks wait in turn).
* ``cp_conv1d``: causal depthwise conv with the k-1 token halo received from the previous rank.

The reference has no sequence parallelism (only a dead ``sequence_parallel`` flag, ``model_zoo.py:79``); these follow
the chunked structure its SSD and flash kernels already have. Collectives go through ``torch.distributed`` (NCCL on
GPUs, gloo in the CPU tests); the tensors exchanged are small next to the attention / scan work they unlock.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import functional as F_
from ..ops import ssm


def _world(group):
    return dist.get_world_size(group), dist.get_rank(group)


class _AllGatherSeq(torch.autograd.Function):
    """[B, Sl, ...] -> [w, B, Sl, ...]; backward sums the gradient slices that the other ranks hold for this shard."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        w, _ = _world(group)
        x = x.contiguous()
        out = x.new_empty((w,) + tuple(x.shape))
        dist.all_gather_into_tensor(out.view(-1), x.view(-1), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        w, r = _world(ctx.group)
        g = g.contiguous()
        if g.is_cuda:
            out = g.new_empty(g.shape[1:])
            dist.reduce_scatter_tensor(out.view(-1), g.view(-1), group=ctx.group)
            return out, None
        dist.all_reduce(g, group=ctx.group)  # gloo has no reduce-scatter
        return g[r].clone(), None


def all_gather_seq(x, group=None):
    return _AllGatherSeq.apply(x, group)


def zigzag_split(x, world: int, rank: int, dim: int = 1):
    """The zigzag shard of a full sequence: chunks `rank` and `2 * world - 1 - rank` of 2 * world equal chunks."""
    c = x.chunk(2 * world, dim=dim)
    return torch.cat([c[rank], c[2 * world - 1 - rank]], dim=dim)


def zigzag_merge(shards, dim: int = 1):
    """Inverse of ``zigzag_split`` given every rank's shard in rank order."""
    w = len(shards)
    parts = [None] * (2 * w)
    for r, s in enumerate(shards):
        a, b = s.chunk(2, dim=dim)
        parts[r], parts[2 * w - 1 - r] = a, b
    return torch.cat(parts, dim=dim)


def cp_attention(q, k, v, causal: bool = True, scale: Optional[float] = None, group=None, layout: str = "contiguous"):
    """q [B, Sl, Hq, D], k / v [B, Sl, Hk, D]: this rank's tokens. Returns the attention output for those tokens.

    contiguous: rank r holds tokens [r * Sl, (r + 1) * Sl). zigzag: see ``zigzag_split`` (Sl must be even).
    """
    w, r = _world(group)
    if w == 1:
        return F_.attention(q, k, v, causal=causal, scale=scale)
    # one collective for K and V (packed along the head axis): half the launches, and one backward reduce-scatter whose
    # order relative to other collectives is the same on every rank
    Hk = k.shape[2]
    kvg = all_gather_seq(torch.cat([k, v], dim=2), group)  # [w, B, Sl, Hk + Hv, D]
    kg, vg = kvg[:, :, :, :Hk], kvg[:, :, :, Hk:]
    B, Sl = q.shape[0], q.shape[1]
    if layout == "contiguous":
        kf = kg.transpose(0, 1).reshape(B, w * Sl, *k.shape[2:])
        vf = vg.transpose(0, 1).reshape(B, w * Sl, *v.shape[2:])
        if not causal:
            return F_.attention(q, kf, vf, causal=False, scale=scale)
        vis = (r + 1) * Sl
        return F_.attention(q, kf[:, :vis], vf[:, :vis], causal=True, scale=scale)
    if layout != "zigzag":
        raise ValueError(f"unknown layout {layout!r}")
    kf = zigzag_merge([kg[i] for i in range(w)])
    vf = zigzag_merge([vg[i] for i in range(w)])
    if not causal:
        return F_.attention(q, kf, vf, causal=False, scale=scale)
    c = Sl // 2
    outs = []
    for half, chunk_id in ((q[:, :c], r), (q[:, c:], 2 * w - 1 - r)):
        vis = (chunk_id + 1) * c
        outs.append(F_.attention(half, kf[:, :vis], vf[:, :vis], causal=True, scale=scale))
    return torch.cat(outs, dim=1)


def merge_attention_blocks(o1, lse1, o2, lse2):
    """Combine two partial attention results over disjoint key sets. o [B, S, H, D], lse [B, H, S]."""
    lse = torch.logaddexp(lse1, lse2)
    w1 = torch.exp(lse1 - lse).transpose(1, 2).unsqueeze(-1)
    w2 = torch.exp(lse2 - lse).transpose(1, 2).unsqueeze(-1)
    w1, w2 = torch.nan_to_num(w1), torch.nan_to_num(w2)  # rows that saw no key in either block
    return (o1.float() * w1 + o2.float() * w2), lse


@torch.no_grad()
def ring_attention_forward(q, k, v, causal: bool = True, scale: Optional[float] = None, group=None):
    """Inference ring attention (contiguous layout). Step s works on the K/V block that started on rank r - s while
    the next block is in flight; blocks from later ranks are skipped under the causal mask."""
    w, r = _world(group)
    o, lse = F_.attention_with_lse(q, k, v, causal=causal, scale=scale)
    o = o.float()
    kb, vb = k.contiguous(), v.contiguous()
    for s in range(1, w):
        send_to, recv_from = (r + 1) % w, (r - 1) % w
        kn, vn = torch.empty_like(kb), torch.empty_like(vb)
        ops = [dist.P2POp(dist.isend, kb, send_to, group), dist.P2POp(dist.isend, vb, send_to, group),
               dist.P2POp(dist.irecv, kn, recv_from, group), dist.P2POp(dist.irecv, vn, recv_from, group)]
        for req in dist.batch_isend_irecv(ops):
            req.wait()
        kb, vb = kn, vn
        src = (r - s) % w
        if causal and src > r:
            continue
        ob, lb = F_.attention_with_lse(q, kb, vb, causal=False, scale=scale)
        o, lse = merge_attention_blocks(o, lse, ob, lb)
    return o.to(q.dtype)


def _ring_rotate(tensors, group):
    """Every tensor goes to rank r + 1 and is replaced by the one arriving from rank r - 1 (one batched exchange)."""
    w, r = _world(group)
    send_to, recv_from = (r + 1) % w, (r - 1) % w
    src = [t.contiguous() for t in tensors]
    dst = [torch.empty_like(t) for t in src]
    ops = [dist.P2POp(dist.isend, t, send_to, group) for t in src] + [dist.P2POp(dist.irecv, t, recv_from, group) for t in dst]
    for req in dist.batch_isend_irecv(ops):
        req.wait()
    return dst


class _RingAttention(torch.autograd.Function):
    """Ring attention with a backward pass (contiguous layout). Forward: K/V blocks travel around the ring and the
    per-block results are merged through their log-sum-exps. Backward: the blocks travel again, each together with
    an accumulator for its dK / dV; every rank adds the contribution of its queries (computed from the FINAL output
    and log-sum-exp, so that the block probabilities are those of the full softmax) and after ``world`` rotations
    every accumulator is back on the rank that owns the block."""

    @staticmethod
    def forward(ctx, q, k, v, causal, scale, group):
        w, r = _world(group)
        o, lse = F_.attention_with_lse(q, k, v, causal=causal, scale=scale)
        o = o.float()
        kb, vb = k.contiguous(), v.contiguous()
        for s in range(1, w):
            kb, vb = _ring_rotate([kb, vb], group)
            if causal and (r - s) % w > r:
                continue
            ob, lb = F_.attention_with_lse(q, kb, vb, causal=False, scale=scale)
            o, lse = merge_attention_blocks(o, lse, ob, lb)
        o = o.to(q.dtype)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.meta = (causal, scale, group)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        causal, scale, group = ctx.meta
        w, r = _world(group)
        do = do.contiguous()
        dq = torch.zeros_like(q, dtype=torch.float32)
        kb, vb = k.contiguous(), v.contiguous()
        dkb, dvb = torch.zeros_like(k, dtype=torch.float32), torch.zeros_like(v, dtype=torch.float32)
        for s in range(w):
            if not (causal and (r - s) % w > r):
                dq_b, dk_b, dv_b = F_.attention_backward(q, kb, vb, o, lse, do, causal=causal and s == 0, window=0,
                                                         scale=scale)
                dq += dq_b.float()
                dkb += dk_b.float()
                dvb += dv_b.float()
            if s + 1 < w:
                kb, vb, dkb, dvb = _ring_rotate([kb, vb, dkb, dvb], group)
            elif w > 1:
                dkb, dvb = _ring_rotate([dkb, dvb], group)      # the last hop brings the accumulators home
        return dq.to(q.dtype), dkb.to(k.dtype), dvb.to(v.dtype), None, None, None


def ring_attention(q, k, v, causal: bool = True, scale: Optional[float] = None, group=None):
    """Ring attention for training over a sequence sharded in contiguous blocks: q, k, v are this rank's
    [B, S / world, H, D] shards; returns this rank's output shard, differentiable in q, k and v."""
    return _RingAttention.apply(q, k, v, causal, scale, group)


# ------------------------------------------------------------------------------------------------ Mamba-2 / SSD
class _SendRecvState(torch.autograd.Function):
    """Forward: send `t` to `dst` (if any) and receive a same-shaped tensor from `src` (if any). Backward mirrors it:
    the gradient of what was received goes back to `src`, and the gradient of what was sent arrives from `dst`."""

    @staticmethod
    def forward(ctx, t, src, dst, group):
        ctx.src, ctx.dst, ctx.group = src, dst, group
        t = t.contiguous()
        got = torch.zeros_like(t)
        if src is not None:
            dist.recv(got, src, group=group)
        if dst is not None:
            dist.send(t, dst, group=group)
        return got

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        back = torch.zeros_like(g)
        if ctx.dst is not None:
            dist.recv(back, ctx.dst, group=ctx.group)
        if ctx.src is not None:
            dist.send(g, ctx.src, group=ctx.group)
        return back, None, None, None


def cp_conv1d(x, w_, bias=None, act=True, group=None):
    """Causal depthwise conv over a sharded sequence: the last k-1 tokens of rank r-1 are the left context of rank r."""
    w, r = _world(group)
    K = w_.shape[1]
    if w == 1:
        return ssm.causal_conv1d(x, w_, bias, act)
    tail = x[:, -(K - 1):].contiguous()
    prev = _exchange_halo(tail, r, w, group)
    return ssm.causal_conv1d(x, w_, bias, act, prev=prev)


class _Halo(torch.autograd.Function):
    """Every rank sends its tail to rank + 1 and receives rank - 1's (rank 0 gets zeros); backward sends the halo
    gradient back. Even ranks send first, odd ranks receive first, so blocking transports do not deadlock."""

    @staticmethod
    def forward(ctx, tail, r, w, group):
        ctx.r, ctx.w, ctx.group = r, w, group
        return _Halo._shift(tail, r, w, group, +1)

    @staticmethod
    def backward(ctx, g):
        return _Halo._shift(g.contiguous(), ctx.r, ctx.w, ctx.group, -1), None, None, None

    @staticmethod
    def _shift(t, r, w, group, direction):
        dst, src = r + direction, r - direction
        got = torch.zeros_like(t)
        send = lambda: dist.send(t, dst, group=group) if 0 <= dst < w else None
        recv = lambda: dist.recv(got, src, group=group) if 0 <= src < w else None
        if r % 2 == 0:
            send()
            recv()
        else:
            recv()
            send()
        return got


def _exchange_halo(tail, r, w, group):
    return _Halo.apply(tail, r, w, group)


def cp_ssd_scan(x, dt, A, Bm, Cm, D=None, chunk=64, group=None, mode: str = "parallel"):
    """SSD scan of a sequence sharded over the group (contiguous layout). Arguments as ``ops.ssm.ssd_scan`` for the
    local tokens; returns the local outputs. See the module docstring for the two modes."""
    w, r = _world(group)
    if w == 1:
        return ssm.ssd_scan(x, dt, A, Bm, Cm, D, chunk)
    if mode == "serial":
        B, _, H, P = x.shape
        N = Bm.shape[-1]
        # requires_grad so that autograd calls the backward that returns the state gradient to the previous rank
        zero = torch.zeros(B, H, P, N, dtype=torch.float32, device=x.device, requires_grad=True)
        init = _SendRecvState.apply(zero, r - 1 if r > 0 else None, None, group) if r > 0 else None
        y, final = ssm.ssd_scan(x, dt, A, Bm, Cm, D, chunk, init_state=init, return_state=True)
        if r + 1 < w:
            token = _SendRecvState.apply(final.float(), None, r + 1, group)  # zeros; keeps the send in the graph
            y = y + token.sum().to(y.dtype) * 0
        return y
    if mode != "parallel":
        raise ValueError(f"unknown mode {mode!r}")
    # pass 1: local final state from a zero initial state, and the shard's total decay per (batch, head)
    _, f_local = ssm.ssd_scan(x, dt, A, Bm, Cm, None, chunk, return_state=True)
    decay_local = torch.exp((dt.float() * A.float().view(1, 1, -1)).sum(1))          # [B, H]
    B, H, P, N = f_local.shape
    # state and decay travel in one packed tensor: one collective forward, one backward, on every rank alike
    packed = all_gather_seq(torch.cat([f_local.float().reshape(B, H, P * N), decay_local.unsqueeze(-1)], dim=-1), group)
    states, decays = packed[..., : P * N].reshape(w, B, H, P, N), packed[..., P * N]
    init = torch.zeros_like(states[0])
    for j in range(r):  # h_r = sum_j F_j * prod_{j < i < r} decay_i, built left to right
        init = init * decays[j][..., None, None] + states[j]
    # pass 2: the scan with the true initial state
    y = ssm.ssd_scan(x, dt, A, Bm, Cm, D, chunk, init_state=init if r > 0 else None)
    # ranks whose output does not use the gathered states (rank 0, and every rank for its successors' entries) still
    # have to take part in the backward collective that returns the other ranks' state gradients
    return y + (packed.sum() * 0).to(y.dtype)


# ----------------------------------------------------------------------------------------------- Ulysses
def _a2a(x, group):
    x = x.contiguous()                 # before empty_like: a permuted view would hand its strides to the output
    out = torch.empty_like(x)
    dist.all_to_all_single(out, x, group=group)
    return out


class _SeqToHead(torch.autograd.Function):
    """[B, S/w, H, D] sharded by sequence -> [B, S, H/w, D] sharded by heads, one all-to-all; backward is the inverse."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _seq_to_head(x, group)

    @staticmethod
    def backward(ctx, g):
        return _head_to_seq(g, ctx.group), None


class _HeadToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _head_to_seq(x, group)

    @staticmethod
    def backward(ctx, g):
        return _seq_to_head(g, ctx.group), None


def _seq_to_head(x, group):
    w = _world(group)[0]
    B, Sl, H, D = x.shape
    send = x.reshape(B, Sl, w, H // w, D).permute(2, 0, 1, 3, 4)            # [head chunk = destination, B, Sl, H/w, D]
    recv = _a2a(send, group)                                                # [source = sequence chunk, B, Sl, H/w, D]
    return recv.permute(1, 0, 2, 3, 4).reshape(B, w * Sl, H // w, D)


def _head_to_seq(x, group):
    w = _world(group)[0]
    B, S, Hl, D = x.shape
    send = x.reshape(B, w, S // w, Hl, D).permute(1, 0, 2, 3, 4)            # [sequence chunk = destination, B, Sl, H/w, D]
    recv = _a2a(send, group)                                                # [source = head chunk, B, Sl, H/w, D]
    return recv.permute(1, 2, 0, 3, 4).reshape(B, S // w, w * Hl, D)


def ulysses_attention(q, k, v, causal: bool = True, scale: Optional[float] = None, group=None):
    """Sequence parallelism by head exchange (DeepSpeed-Ulysses): q, k, v arrive sharded along the sequence
    ([B, S/w, H, D], contiguous layout); one all-to-all per tensor turns them into full-sequence tensors holding H/w
    heads, attention runs locally with no further communication, and one all-to-all returns the output to sequence
    shards. Traffic per rank is 4 x (S/w) x H x D elements regardless of S, against the (w-1)/w x S x Hkv x D x 2 of the
    all-gather form, so it wins when Hkv is not much smaller than H; it needs H (and Hkv, after repetition) divisible
    by w. The reference has only the unused ``sequence_parallel`` flag (include/neural_core/architecture/distributed.h)."""
    w = _world(group)[0]
    if w == 1:
        return F_.attention(q, k, v, causal=causal, scale=scale)
    Hq, Hk = q.shape[2], k.shape[2]
    if Hq % w:
        raise ValueError(f"{Hq} query heads cannot be split over {w} ranks")
    if Hk % w:                                      # grouped KV heads that do not divide: expand to one per query head
        k, v = k.repeat_interleave(Hq // Hk, dim=2), v.repeat_interleave(Hq // Hk, dim=2)
    qh, kh, vh = (_SeqToHead.apply(t, group) for t in (q, k, v))
    o = F_.attention(qh, kh, vh, causal=causal, scale=scale)
    return _HeadToSeq.apply(o, group)

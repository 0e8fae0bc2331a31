"""Pipeline parallelism: stages exchange activations / activation gradients with point-to-point sends (NCCL p2p on
GPUs, gloo on CPU ranks) under a 1F1B schedule; sends and receives are posted asynchronously so that they overlap
with the neighbouring micro-batch's compute. The reference describes 1F1B but runs micro-batches sequentially
through 1 MiB staging buffers with no inter-rank traffic (kernel/distributed/pipeline.c:46-136); its stage
callbacks (include/neural_core/architecture/distributed.h:113-122) correspond to ``stage_module`` here.

Stage contract: the first stage's module maps ``input_ids -> hidden``, middle stages ``hidden -> hidden``, the
last stage ``(hidden, labels) -> loss``. Hidden activations are single tensors of a fixed shape per micro-batch.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


class PipelineSchedule:
    """Order of forward (F) / backward (B) micro-batch steps for one stage."""

    @staticmethod
    def one_f_one_b(stage: int, num_stages: int, num_microbatches: int) -> List[tuple]:
        warm = min(num_stages - stage - 1, num_microbatches)
        steps = [("F", i) for i in range(warm)]
        f, b = warm, 0
        while f < num_microbatches:
            steps.append(("F", f))
            steps.append(("B", b))
            f += 1
            b += 1
        while b < num_microbatches:
            steps.append(("B", b))
            b += 1
        return steps

    @staticmethod
    def gpipe(stage: int, num_stages: int, num_microbatches: int) -> List[tuple]:
        return [("F", i) for i in range(num_microbatches)] + [("B", i) for i in range(num_microbatches)]


def plan_rounds(schedules: List[List[tuple]], num_ranks: int, num_chunks: int):
    """Turns the per-rank schedules (lists of (kind, chunk, micro-batch)) into globally agreed communication rounds.

    Every rank runs the same simulation: in a round each rank executes its next step if the message that step
    consumes was produced in an earlier round; the messages produced in a round are exchanged at the round's end, every
    rank issuing ONE batch of sends and receives. Both ends of every pair therefore post their operations in the same
    order, which is what transports without message tags (NCCL matches point-to-point operations of a pair strictly in
    posting order and runs them one after another) need in order not to dead-lock; opposite-direction transfers of a
    round travel in one batch and progress together. Returns, per round, (steps executed per rank, messages
    [(key, src, dst)]), where key = (direction, consuming virtual stage, micro-batch)."""
    P, v = num_ranks, num_chunks
    last_vs = P * v - 1

    def consumes(r, step):
        kind, c, i = step
        vs = c * P + r
        if kind == "F":
            return None if vs == 0 else ("act", vs, i)
        return None if vs == last_vs else ("grad", vs, i)

    def produces(r, step):
        kind, c, i = step
        vs = c * P + r
        if kind == "F":
            return None if vs == last_vs else (("act", vs + 1, i), (vs + 1) % P)
        return None if vs == 0 else (("grad", vs - 1, i), (vs - 1) % P)

    ptr = [0] * P
    avail = set()
    rounds = []
    while any(ptr[r] < len(schedules[r]) for r in range(P)):
        executed = [None] * P
        for r in range(P):
            if ptr[r] < len(schedules[r]):
                need = consumes(r, schedules[r][ptr[r]])
                if need is None or need in avail:
                    executed[r] = schedules[r][ptr[r]]
        if not any(e is not None for e in executed):
            raise RuntimeError("pipeline schedule cannot make progress (a step waits for a message nobody sends)")
        msgs = []
        for r in range(P):
            if executed[r] is not None:
                ptr[r] += 1
                out = produces(r, executed[r])
                if out is not None:
                    msgs.append((out[0], r, out[1]))
        avail.update(k for k, _, _ in msgs)
        rounds.append((executed, msgs))
    return rounds


def run_rounds(rounds, rank: int, group, hidden_shape, dtype, device, forward_step, backward_step):
    """Executes this rank's part of ``plan_rounds``. ``forward_step(chunk, mb, x_or_None) -> tensor to send or None``;
    ``backward_step(chunk, mb, grad_or_None) -> tensor to send or None``."""
    inbox = {}
    P = dist.get_world_size(group)
    glob = [dist.get_global_rank(group, r) for r in range(P)]
    for executed, msgs in rounds:
        outgoing = None
        step = executed[rank]
        if step is not None:
            kind, c, i = step
            vs = c * P + rank
            if kind == "F":
                outgoing = forward_step(c, i, inbox.pop(("act", vs, i), None))
            else:
                outgoing = backward_step(c, i, inbox.pop(("grad", vs, i), None))
        ops, bufs = [], []
        for key, src, dst in msgs:
            if src == rank:
                ops.append(dist.P2POp(dist.isend, outgoing.contiguous(), glob[dst], group))
            if dst == rank:
                buf = torch.empty(hidden_shape, dtype=dtype, device=device)
                bufs.append((key, buf))
                ops.append(dist.P2POp(dist.irecv, buf, glob[src], group))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        for key, buf in bufs:
            inbox[key] = buf


class PipelineStage:
    def __init__(self, stage_module: torch.nn.Module, group=None, hidden_shape=None, dtype=None, device=None,
                 schedule: str = "1f1b"):
        self.module = stage_module
        self.group = group if group is not None else dist.group.WORLD
        self.stage = dist.get_rank(self.group)
        self.num_stages = dist.get_world_size(self.group)
        self.first, self.last = self.stage == 0, self.stage == self.num_stages - 1
        self.hidden_shape, self.dtype, self.device = hidden_shape, dtype, device
        self.schedule = schedule
        self.prev = dist.get_global_rank(self.group, self.stage - 1) if not self.first else None
        self.next = dist.get_global_rank(self.group, self.stage + 1) if not self.last else None

    def forward_backward(self, inputs: Optional[List[torch.Tensor]], labels: Optional[List[torch.Tensor]],
                         num_microbatches: int, loss_scale: Optional[float] = None):
        """Runs all micro-batches of one step. ``inputs`` on the first stage, ``labels`` on the last. Returns the mean
        loss on the last stage (None elsewhere). Gradients accumulate in the stage's parameters. Activations and
        gradients move in globally ordered rounds (``plan_rounds``), one batched send / receive per round, so the same
        code runs on NCCL point-to-point (no tags, strict pairwise order) and on gloo."""
        M, P = num_microbatches, self.num_stages
        make = PipelineSchedule.one_f_one_b if self.schedule == "1f1b" else PipelineSchedule.gpipe
        schedules = [[(k, 0, i) for k, i in make(st, P, M)] for st in range(P)]
        rounds = plan_rounds(schedules, P, 1)
        scale = loss_scale if loss_scale is not None else 1.0 / M
        saved, losses = {}, []

        def fwd(c, i, x):
            x = inputs[i] if self.first else x.requires_grad_(True)
            out = self.module(x, labels[i]) if self.last else self.module(x)
            saved[i] = (x, out)
            if self.last:
                losses.append(out.detach())
                return None
            return out.detach()

        def bwd(c, i, g):
            x, out = saved.pop(i)
            if self.last:
                (out * scale).backward()
            else:
                out.backward(g)
            return None if self.first else x.grad

        run_rounds(rounds, self.stage, self.group, self.hidden_shape, self.dtype, self.device, fwd, bwd)
        return torch.stack(losses).mean() if self.last else None


def split_layers(num_layers: int, num_stages: int) -> List[range]:
    """Contiguous, as-even-as-possible layer ranges per stage (earlier stages take the remainder)."""
    base, rem = divmod(num_layers, num_stages)
    out, s = [], 0
    for i in range(num_stages):
        n = base + (1 if i < rem else 0)
        out.append(range(s, s + n))
        s += n
    return out


class LlamaStage(torch.nn.Module):
    """One pipeline stage of a Llama-family model: optional embedding, a slice of the decoder layers, optional final
    norm + LM head + loss."""

    def __init__(self, full_model, layer_range, first: bool, last: bool):
        super().__init__()
        self.cfg = full_model.config
        self.first, self.last = first, last
        self.embedding = full_model.embedding if first else None
        self.layers = torch.nn.ModuleList([full_model.layers[i] for i in layer_range])
        self.norm = full_model.norm if last else None
        self.head_weight_fn = full_model.head_weight if last else None
        self._full = [full_model]   # kept out of the module tree: only used for the rope tables

    def forward(self, x, labels=None):
        from ..ops import functional as ops
        model = self._full[0]
        if self.first:
            S = x.shape[1]
            h, resid = self.embedding(x), None
        else:
            S = x.shape[1]
            # activations cross stage boundaries as the already-summed residual stream
            h, resid = x, None
        rope = model.rope(x.device, S)
        for layer in self.layers:
            h, resid = layer(h, resid, rope)
        if resid is not None:
            hidden = (h.float() + resid.float()).to(h.dtype)
        else:
            hidden = h
        if not self.last:
            return hidden
        hn = self.norm(hidden)
        tgt = torch.full_like(labels, -100)
        tgt[:, :-1] = labels[:, 1:]
        return ops.linear_cross_entropy(hn, self.head_weight_fn(), tgt)


# ---------------------------------------------------------------------------------------------- interleaved 1F1B
def interleaved_schedule(rank: int, num_ranks: int, num_chunks: int, num_microbatches: int) -> List[tuple]:
    """Steps ("F" | "B", chunk, micro-batch) of one rank under interleaved 1F1B: each rank holds `num_chunks` model
    chunks; virtual stage s = chunk * num_ranks + rank. Micro-batches advance in groups of `num_ranks`, chunk by chunk,
    which shrinks the pipeline bubble by the number of chunks. `num_microbatches` must be a multiple of `num_ranks`."""
    P, v, M = num_ranks, num_chunks, num_microbatches
    if M % P:
        raise ValueError("interleaved schedule needs num_microbatches to be a multiple of the number of ranks")
    total = M * v

    def fwd(k):
        return (k // P) % v, (k // (P * v)) * P + k % P

    def bwd(k):
        c, i = fwd(k)
        return v - 1 - c, i

    warm = min((P - rank - 1) * 2 + (v - 1) * P, total)
    steps = [("F",) + fwd(k) for k in range(warm)]
    f, b = warm, 0
    while f < total:
        steps.append(("F",) + fwd(f))
        steps.append(("B",) + bwd(b))
        f += 1
        b += 1
    while b < total:
        steps.append(("B",) + bwd(b))
        b += 1
    return steps


class InterleavedPipelineStage:
    """Interleaved pipeline over `num_chunks` model chunks per rank. ``chunks[c]`` is the module of virtual stage
    ``c * P + rank``; the very first virtual stage takes ``inputs``, the very last ``(hidden, labels) -> loss``.

    Messages move in the globally ordered rounds of ``plan_rounds`` (one batched send / receive per round and rank),
    which needs no message tags and so also runs on NCCL point-to-point."""

    def __init__(self, chunks: List[torch.nn.Module], group=None, hidden_shape=None, dtype=None, device=None):
        self.chunks = list(chunks)
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.P = dist.get_world_size(self.group)
        self.v = len(self.chunks)
        self.hidden_shape, self.dtype, self.device = hidden_shape, dtype, device
        self.right = dist.get_global_rank(self.group, (self.rank + 1) % self.P)
        self.left = dist.get_global_rank(self.group, (self.rank - 1) % self.P)

    def forward_backward(self, inputs, labels, num_microbatches: int, loss_scale: Optional[float] = None):
        P, v, M = self.P, self.v, num_microbatches
        last_vs = P * v - 1
        scale = loss_scale if loss_scale is not None else 1.0 / M
        rounds = plan_rounds([interleaved_schedule(r, P, v, M) for r in range(P)], P, v)
        saved, losses = {}, []

        def fwd(c, i, x):
            vs = c * P + self.rank
            x = inputs[i] if vs == 0 else x.requires_grad_(True)
            out = self.chunks[c](x, labels[i]) if vs == last_vs else self.chunks[c](x)
            saved[(c, i)] = (x, out)
            if vs == last_vs:
                losses.append(out.detach())
                return None
            return out.detach()

        def bwd(c, i, g):
            vs = c * P + self.rank
            x, out = saved.pop((c, i))
            if vs == last_vs:
                (out * scale).backward()
            else:
                out.backward(g)
            return None if vs == 0 else x.grad

        run_rounds(rounds, self.rank, self.group, self.hidden_shape, self.dtype, self.device, fwd, bwd)
        return torch.stack(losses).mean() if losses else None


def split_layers_interleaved(num_layers: int, num_ranks: int, num_chunks: int) -> List[List[range]]:
    """Layer ranges per rank and chunk: virtual stage c * num_ranks + r gets the (c * num_ranks + r)-th slice."""
    slices = split_layers(num_layers, num_ranks * num_chunks)
    return [[slices[c * num_ranks + r] for c in range(num_chunks)] for r in range(num_ranks)]

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

    def _recv(self, src):
        buf = torch.empty(self.hidden_shape, dtype=self.dtype, device=self.device)
        return buf, dist.irecv(buf, src=src, group=self.group)

    def forward_backward(self, inputs: Optional[List[torch.Tensor]], labels: Optional[List[torch.Tensor]],
                         num_microbatches: int, loss_scale: Optional[float] = None):
        """Runs all micro-batches of one step. ``inputs`` on the first stage, ``labels`` on the last. Returns the mean
        loss on the last stage (None elsewhere). Gradients accumulate in the stage's parameters."""
        M = num_microbatches
        sched = (PipelineSchedule.one_f_one_b if self.schedule == "1f1b" else PipelineSchedule.gpipe)(
            self.stage, self.num_stages, M)
        scale = loss_scale if loss_scale is not None else 1.0 / M
        saved_in, saved_out = {}, {}
        pending_sends = []
        losses = []
        # post the first receive early; later ones are posted one step ahead so they overlap with compute
        next_fwd_recv = self._recv(self.prev) if not self.first else None
        next_bwd_recv = None
        fwd_seen = 0
        for kind, i in sched:
            if kind == "F":
                if self.first:
                    x = inputs[i]
                else:
                    buf, work = next_fwd_recv
                    work.wait()
                    fwd_seen += 1
                    next_fwd_recv = self._recv(self.prev) if fwd_seen < M else None
                    x = buf.requires_grad_(True)
                if self.last:
                    out = self.module(x, labels[i])
                    losses.append(out.detach())
                    saved_out[i] = out
                else:
                    out = self.module(x)
                    pending_sends.append(dist.isend(out.detach().contiguous(), dst=self.next, group=self.group))
                    saved_out[i] = out
                    if next_bwd_recv is None:
                        next_bwd_recv = self._recv(self.next)
                saved_in[i] = x
            else:
                x, out = saved_in.pop(i), saved_out.pop(i)
                if self.last:
                    (out * scale).backward()
                else:
                    gbuf, work = next_bwd_recv
                    work.wait()
                    next_bwd_recv = self._recv(self.next) if any(k == "B" and j > i for k, j in sched) else None
                    out.backward(gbuf)
                if not self.first:
                    pending_sends.append(dist.isend(x.grad.contiguous(), dst=self.prev, group=self.group))
        for w in pending_sends:
            w.wait()
        if self.last:
            return torch.stack(losses).mean()
        return None


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

    Messages carry a tag derived from (direction, virtual stage, micro-batch): transports that match on tags (gloo)
    pair them regardless of posting order. Sends are asynchronous and receives are posted when their step comes up, so
    the only waits are the data dependencies of the schedule."""

    def __init__(self, chunks: List[torch.nn.Module], group=None, hidden_shape=None, dtype=None, device=None):
        self.chunks = list(chunks)
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.P = dist.get_world_size(self.group)
        self.v = len(self.chunks)
        self.hidden_shape, self.dtype, self.device = hidden_shape, dtype, device
        self.right = dist.get_global_rank(self.group, (self.rank + 1) % self.P)
        self.left = dist.get_global_rank(self.group, (self.rank - 1) % self.P)

    def _tag(self, backward: bool, vstage: int, mb: int) -> int:
        return (1 << 20) * int(backward) + vstage * 1024 + mb

    def forward_backward(self, inputs, labels, num_microbatches: int, loss_scale: Optional[float] = None):
        P, v, M = self.P, self.v, num_microbatches
        last_vs = P * v - 1
        scale = loss_scale if loss_scale is not None else 1.0 / M
        saved, sends, losses = {}, [], []
        for kind, c, i in interleaved_schedule(self.rank, P, v, M):
            vs = c * P + self.rank
            if kind == "F":
                if vs == 0:
                    x = inputs[i]
                else:
                    x = torch.empty(self.hidden_shape, dtype=self.dtype, device=self.device)
                    dist.recv(x, src=self.left, group=self.group, tag=self._tag(False, vs, i))
                    x.requires_grad_(True)
                if vs == last_vs:
                    out = self.chunks[c](x, labels[i])
                    losses.append(out.detach())
                else:
                    out = self.chunks[c](x)
                    sends.append(dist.isend(out.detach().contiguous(), dst=self.right, group=self.group,
                                            tag=self._tag(False, vs + 1, i)))
                saved[(c, i)] = (x, out)
            else:
                x, out = saved.pop((c, i))
                if vs == last_vs:
                    (out * scale).backward()
                else:
                    g = torch.empty_like(out)
                    dist.recv(g, src=self.right, group=self.group, tag=self._tag(True, vs, i))
                    out.backward(g)
                if vs != 0:
                    sends.append(dist.isend(x.grad.contiguous(), dst=self.left, group=self.group,
                                            tag=self._tag(True, vs - 1, i)))
        for w in sends:
            w.wait()
        return torch.stack(losses).mean() if losses else None


def split_layers_interleaved(num_layers: int, num_ranks: int, num_chunks: int) -> List[List[range]]:
    """Layer ranges per rank and chunk: virtual stage c * num_ranks + r gets the (c * num_ranks + r)-th slice."""
    slices = split_layers(num_layers, num_ranks * num_chunks)
    return [[slices[c * num_ranks + r] for c in range(num_chunks)] for r in range(num_ranks)]

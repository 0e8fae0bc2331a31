"""Pipeline parallelism: stages exchange activations / activation gradients with point-to-point sends (NCCL p2p on
GPUs, gloo on CPU ranks) under a 1F1B schedule; sends and receives are posted asynchronously so that they overlap
with the neighbouring micro-batch's compute. The reference describes 1F1B but runs micro-batches sequentially
through 1 MiB staging buffers with no inter-rank traffic (kernel/distributed/pipeline.c:46-136); its stage
callbacks (include/neural_core/architecture/distributed.h:113-122) correspond to ``stage_module`` here.

Stage contract: the first stage's module maps ``input_ids -> hidden``, middle stages ``hidden -> hidden``, the
last stage ``(hidden, labels) -> loss``. Hidden activations are single tensors of a fixed shape per micro-batch.
"""
from __future__ import annotations

from typing import Callable, List, Optional

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

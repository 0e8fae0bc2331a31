"""Flat-buffer training engine: every parameter lives in one contiguous bf16 buffer, every gradient
in one contiguous buffer that the wgrad GEMMs write directly (``main_grad`` views), and the whole
optimizer step is three launches (norm partials, norm finalise, fused AdamW).

With one process this is the degenerate (world size 1) case of the ZeRO engine in
``parallel/zero.py``, which shards the same flat buffers. The reference's counterparts are the C
trainer step (kernel/train/trainer.c:114-203) and ``Trainer.train_step``
(interface_bindings/trainer_v3.py:439).
"""
from __future__ import annotations

from typing import Iterable, List, Optional

import torch

from ..optim.fused import adamw_flat_, grad_norm_


def _unique_params(module) -> List[torch.nn.Parameter]:
    seen, out = set(), []
    for p in module.parameters():
        if p.requires_grad and id(p) not in seen:
            seen.add(id(p))
            out.append(p)
    return out


class FlatParams:
    """Re-homes the parameters of ``module`` into one flat buffer and gives each a ``main_grad`` view
    into one flat gradient buffer. ``align`` pads every tensor so that views stay 16-byte aligned and
    the total is divisible by ``shard_multiple`` (so it splits evenly across ranks). ``group_starts`` lists the
    indices of parameters that open a bucket: their offsets are rounded up to ``align * shard_multiple`` so every
    bucket splits evenly too, whatever the sizes of the tensors inside it."""

    def __init__(self, module, grad_dtype: Optional[torch.dtype] = None, align: int = 64, shard_multiple: int = 1,
                 params: Optional[Iterable[torch.nn.Parameter]] = None, alloc=None, group_starts=()):
        self.params = list(params) if params is not None else _unique_params(module)
        assert self.params, "no trainable parameters"
        p0 = self.params[0]
        # one storage dtype for the whole buffer: the widest-used 16-bit type if any parameter has one (fp32
        # scalars such as SSM decay rates are then computed from their fp32 master copy, rounded for the forward pass)
        dts = {p.dtype for p in self.params}
        self.dtype = torch.bfloat16 if torch.bfloat16 in dts else (torch.float16 if torch.float16 in dts else p0.dtype)
        self.device = p0.device
        self.grad_dtype = grad_dtype or self.dtype
        self.offsets = []
        off = 0
        unit = align * shard_multiple
        starts = set(group_starts)
        for i, p in enumerate(self.params):
            assert p.device == self.device
            if i in starts:
                off = (off + unit - 1) // unit * unit
            self.offsets.append(off)
            off += (p.numel() + align - 1) // align * align
        self.total = (off + unit - 1) // unit * unit
        alloc = alloc or (lambda n, dt: torch.zeros(n, dtype=dt, device=self.device))
        self.flat = alloc(self.total, self.dtype)
        self.grad = alloc(self.total, self.grad_dtype)
        with torch.no_grad():
            for p, o in zip(self.params, self.offsets):
                view = self.flat[o: o + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
                p.main_grad = self.grad[o: o + p.numel()].view(p.shape)
                p._main_grad_written = False

    def begin_step(self):
        for p in self.params:
            p._main_grad_written = False
            p.grad = None

    @torch.no_grad()
    def finalize_grads(self):
        """Fold autograd-produced ``.grad`` tensors into the flat buffer and zero what nothing wrote."""
        for p in self.params:
            if p.grad is not None:
                if p._main_grad_written:
                    p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                else:
                    p.main_grad.copy_(p.grad)
                p._main_grad_written = True
                p.grad = None
            elif not p._main_grad_written:
                p.main_grad.zero_()


class TrainEngine:
    """Single-process engine: forward/backward through the model's own loss, then the fused step."""

    def __init__(self, model, lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, max_grad_norm=1.0,
                 grad_dtype=None):
        self.model = model
        self.fp = FlatParams(model, grad_dtype=grad_dtype)
        self.master = self.fp.flat.float()
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.max_grad_norm = max_grad_norm
        self.step_count = 0
        self.last_norm = None

    def forward_backward(self, input_ids, labels, **kw):
        self.fp.begin_step()
        out = self.model(input_ids, labels=labels, **kw)
        loss = out["loss"] if isinstance(out, dict) else out
        loss.backward()
        self.fp.finalize_grads()
        return loss.detach()

    def optimizer_step(self):
        self.step_count += 1
        out, flag = grad_norm_([self.fp.grad], self.max_grad_norm)
        self.last_norm = out
        p16 = self.fp.flat if self.fp.flat.dtype != torch.float32 else None
        target = self.master if p16 is not None else self.fp.flat
        adamw_flat_(target, self.m, self.v, self.fp.grad, p16, self.lr, self.betas[0], self.betas[1], self.eps,
                    self.wd, self.step_count, 1.0, out[2:3])
        if p16 is None and self.master is not self.fp.flat:
            self.master = self.fp.flat

    def step(self, input_ids, labels, **kw):
        loss = self.forward_backward(input_ids, labels, **kw)
        self.optimizer_step()
        return loss

    def state_dict(self):
        return {"step": self.step_count, "master": self.master, "m": self.m, "v": self.v}

    def load_state_dict(self, sd):
        self.step_count = int(sd["step"])
        self.master.copy_(sd["master"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        self.fp.flat.copy_(self.master)

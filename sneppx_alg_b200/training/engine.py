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
    """Single-process engine: forward/backward through the model's own loss, then the fused step.

    On a GPU the AdamW update is issued per bucket (what runs before the layers, each layer, what runs after them) in
    forward order on a side stream, and the next forward pass waits for a bucket only when it reaches it: the update
    is bound by memory bandwidth, the forward GEMMs by the tensor cores, so most of the 28 bytes per parameter move
    while the next step is already computing. The gradient norm (and with it the clip coefficient) is still computed
    from all gradients before any parameter changes. ``finish()`` makes the calling stream wait for updates still
    in flight; ``state_dict`` / ``load_state_dict`` call it. ``overlap_optimizer=False`` keeps everything on one
    stream."""

    def __init__(self, model, lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, max_grad_norm=1.0,
                 grad_dtype=None, overlap_optimizer=None):
        self.model = model
        self.fp = FlatParams(model, grad_dtype=grad_dtype)
        self.master = self.fp.flat.float()
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.max_grad_norm = max_grad_norm
        self.step_count = 0
        self.last_norm = None
        self._ranges, self._events, self._opt_stream = None, [], None
        cuda = self.fp.device.type == "cuda"
        if (overlap_optimizer if overlap_optimizer is not None else cuda) and cuda and self.fp.flat.dtype != torch.float32:
            self._setup_overlap()

    # ------------------------------------------------------------------ optimizer overlap
    def _setup_overlap(self):
        """Bucket ranges of the flat buffer in forward order and the hooks that wait for their updates."""
        from ..parallel.zero_engine import _find_layer_list
        layers = _find_layer_list(self.model)
        if layers is None or len(layers) == 0:
            return
        index = {id(p): i for i, p in enumerate(self.fp.params)}
        ends = [o + (p.numel() + 63) // 64 * 64 for p, o in zip(self.fp.params, self.fp.offsets)]
        spans = []
        for layer in layers:
            ids = sorted(index[id(p)] for p in layer.parameters() if id(p) in index)
            if not ids or ids != list(range(ids[0], ids[-1] + 1)):
                return                       # a layer whose parameters are not one contiguous run: keep one stream
            spans.append((self.fp.offsets[ids[0]], ends[ids[-1]]))
        if any(spans[i][1] > spans[i + 1][0] for i in range(len(spans) - 1)):
            return
        ranges = [(0, spans[0][0])] + [(spans[i][0], spans[i + 1][0] if i + 1 < len(spans) else spans[i][1])
                                       for i in range(len(spans))] + [(spans[-1][1], self.fp.total)]
        self._ranges = ranges                # [pre, layer 0, .., layer L-1, post]; empty ranges are skipped
        self._events = [None] * len(ranges)
        self._opt_stream = torch.cuda.Stream(device=self.fp.device)
        eng = self

        def waiter(bi):
            def pre(mod, args):
                eng._wait(bi)
            return pre

        for i, layer in enumerate(layers):
            layer.register_forward_pre_hook(waiter(i + 1))
        layers[-1].register_forward_hook(lambda mod, args, out: eng._wait(len(ranges) - 1))

    def _wait(self, bi):
        ev = self._events[bi] if self._events else None
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
            self._events[bi] = None

    def finish(self):
        """The calling stream waits for every parameter update issued so far."""
        if self._opt_stream is not None:
            torch.cuda.current_stream().wait_stream(self._opt_stream)
            self._events = [None] * len(self._events)

    def forward_backward(self, input_ids, labels, **kw):
        self._wait(0)                        # embeddings (and whatever else runs before the layers)
        self.fp.begin_step()
        out = self.model(input_ids, labels=labels, **kw)
        loss = out["loss"] if isinstance(out, dict) else out
        loss.backward()
        self.fp.finalize_grads()
        return loss.detach()

    def optimizer_step(self):
        self.step_count += 1
        # updates of the previous step that no forward hook waited for (a layer that was skipped) end here; this also
        # keeps the clip coefficient they read (a reused scratch tensor) alive until they are done
        self.finish()
        out, flag = grad_norm_([self.fp.grad], self.max_grad_norm)
        self.last_norm = out
        p16 = self.fp.flat if self.fp.flat.dtype != torch.float32 else None
        target = self.master if p16 is not None else self.fp.flat
        if self._opt_stream is not None:
            side = self._opt_stream
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for bi, (b0, b1) in enumerate(self._ranges):
                    if b1 > b0:
                        adamw_flat_(self.master[b0:b1], self.m[b0:b1], self.v[b0:b1], self.fp.grad[b0:b1],
                                    self.fp.flat[b0:b1], self.lr, self.betas[0], self.betas[1], self.eps, self.wd,
                                    self.step_count, 1.0, out[2:3])
                        ev = torch.cuda.Event()
                        ev.record(side)
                        self._events[bi] = ev
            return
        adamw_flat_(target, self.m, self.v, self.fp.grad, p16, self.lr, self.betas[0], self.betas[1], self.eps,
                    self.wd, self.step_count, 1.0, out[2:3])
        if p16 is None and self.master is not self.fp.flat:
            self.master = self.fp.flat

    def step(self, input_ids, labels, **kw):
        loss = self.forward_backward(input_ids, labels, **kw)
        self.optimizer_step()
        return loss

    def state_dict(self):
        self.finish()
        return {"step": self.step_count, "master": self.master, "m": self.m, "v": self.v}

    def load_state_dict(self, sd):
        self.finish()
        self.step_count = int(sd["step"])
        self.master.copy_(sd["master"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        self.fp.flat.copy_(self.master)

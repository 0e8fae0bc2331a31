"""ZeRO-1/2/3 data-parallel engine over bucketed flat buffers.

Partitioning: the model's parameters are laid out bucket by bucket (one bucket per repeated layer, one for
everything else) in a flat bf16 buffer; each bucket is split evenly over the ranks, so rank r owns the r-th
slice of every bucket: fp32 master weights, both Adam moments and the bf16 parameter shard that peers gather
from. (The reference splits one flat vector with the first ``n % w`` ranks taking one extra element,
kernel/distributed/zero.c:53-66, interface_bindings/fsdp.py:40-54; here buckets are padded to a multiple of
64 elements instead so that every slice is 16-byte aligned. ``partition_range`` keeps the reference rule for
callers that want it.)

Fused path (CUDA, symmetric memory): as soon as the backward pass finishes a bucket, ``sx_zero_step`` (mode 1)
reduces this rank's slice straight out of every peer's gradient buffer on a side stream, overlapped with the rest
of backward; after the last bucket one more launch (mode 2) exchanges the squared norms, clips and applies AdamW
to the shard; parameters for the next step are pulled bucket by bucket over NVLink ahead of the layer that needs
them. Stage 1 reduces once at the end of backward, stage 2 reduces per bucket, stage 3 additionally treats the
full bf16 parameter buffer as a cache that is refilled from the owners' shards every step.

Sharded parameters (``param_slots=K``, stage 3 only): the gathered bf16 parameters of the repeated layers are not
kept. ``K`` layer-sized slots rotate: layer i lives in slot i mod K, is gathered K - 1 layers ahead of its forward
pass, overwritten by layer i + K once its forward is done, and gathered again ahead of its backward pass (the
parameters of every layer alias the slot memory, so tensors saved for backward see the right values again). Per GPU
this keeps K layers plus the embedding / head bucket instead of the whole model, at the price of a second all-gather
of the layers per step. (The reference's FSDP wrapper describes the same ``FULL_SHARD`` behaviour,
interface_bindings/fsdp.py:132-151,187-194.)

Library path (``fused=False``, also CPU/gloo): ``reduce_scatter`` / ``all_reduce`` / ``all_gather`` from
``torch.distributed`` around the same local math. This is the baseline the fused path is measured against.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List

import torch
import torch.distributed as dist

from ..ops import _lib
from ..optim.fused import adamw_flat_, grad_norm_
from ..training.engine import FlatParams, _unique_params


def partition_range(n: int, world: int, rank: int):
    """Reference partition rule: first ``n % world`` ranks get one extra element (zero.c:53-66)."""
    base, rem = divmod(n, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def _find_layer_list(model):
    best = None
    for mod in model.modules():
        if isinstance(mod, torch.nn.ModuleList) and len(mod) > 1:
            if best is None or len(mod) > len(best):
                best = mod
    return best


class ZeroEngine:
    def __init__(self, model, zero_stage=3, lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1,
                 max_grad_norm=1.0, group=None, fused=None, comm_grid=0, timeout_s=5.0, nvls=None, param_slots=None):
        self.model = model
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.stage = zero_stage
        self.lr, self.betas, self.eps, self.wd, self.max_grad_norm = lr, betas, eps, weight_decay, max_grad_norm
        self.step_count = 0
        # Expert weights of an expert-parallel model (``is_expert``) differ between ranks: they are not reduced or
        # partitioned over the data-parallel group; this rank keeps their full optimizer state and updates them locally.
        self.expert_params = [p for p in _unique_params(model) if getattr(p, "is_expert", False)]
        params = [p for p in _unique_params(model) if not getattr(p, "is_expert", False)]
        dev = params[0].device
        self.device = dev
        self.fused = (dev.type == "cuda" and params[0].dtype == torch.bfloat16) if fused is None else fused
        # NVLS (in-switch reduction / multicast stores) for the gradient reduce-scatter and the parameter
        # all-gather; needs a multicast mapping of the symmetric buffers, else the peer-load kernels run.
        if nvls is None:
            nvls = os.environ.get("SX_ZERO_NVLS", "0") == "1"
        self.nvls = bool(nvls) and self.fused
        if param_slots is None:
            param_slots = int(os.environ.get("SX_ZERO_PARAM_SLOTS", "0"))
        self.param_slots = int(param_slots) if zero_stage >= 3 else 0
        if self.param_slots:
            assert self.param_slots >= 2, "at least two slots (one in use, one being filled)"
            assert not self.nvls, "sharded parameters use the peer-load all-gather"
        # ---- buckets: one per repeated layer (in forward order), then what runs before the layers (embedding) and
        # what runs after them (final norm, head): the last group's gradients are complete first in backward
        layers = _find_layer_list(model)
        bucket_params: List[List[torch.nn.Parameter]] = []
        taken = set()
        self.bucket_modules = []
        if layers is not None:
            for layer in layers:
                ps = [p for p in _unique_params(layer) if id(p) not in taken and not getattr(p, "is_expert", False)]
                if ps:
                    taken.update(id(p) for p in ps)
                    bucket_params.append(ps)
                    self.bucket_modules.append(layer)
        rest = [p for p in params if id(p) not in taken]
        self.rest_index = len(bucket_params)      # first of the non-layer buckets
        self.post_index = None
        if rest and layers is not None:
            # parameters registered after the layer list are used after it in forward (final norm, untied head)
            order = [id(p) for _, p in model.named_parameters()]
            layer_ids = {id(p) for l in layers for p in l.parameters()}
            first_layer = min((i for i, q in enumerate(order) if q in layer_ids), default=len(order))
            pos = {q: i for i, q in enumerate(order)}
            pre = [p for p in rest if pos.get(id(p), 0) < first_layer]
            post = [p for p in rest if pos.get(id(p), 0) >= first_layer]
            if pre and post:
                bucket_params.append(pre)
                self.post_index = len(bucket_params)
                bucket_params.append(post)
            else:
                bucket_params.append(rest)
        elif rest:
            bucket_params.append(rest)
        ordered = [p for b in bucket_params for p in b]
        self.sg = None
        alloc = None
        self._symm = {}
        if self.fused:
            from .symm import SymmGroup
            self.sg = SymmGroup(self.group, timeout_s=timeout_s)
            calls = []

            def alloc(n, dt):
                # FlatParams asks for the parameter buffer first, then the gradient buffer. Gradients must be
                # peer-readable (owners pull their slice from every rank); gathered parameters are local, unless
                # they are filled by multicast stores (NVLS), which need the symmetric mapping too.
                calls.append(n)
                if len(calls) == 2 or (len(calls) == 1 and self.nvls):
                    b = self.sg.alloc(n, dt)
                    self._symm["grad" if len(calls) == 2 else "param"] = b
                    b.tensor.zero_()
                    return b.tensor
                return torch.zeros(n, dtype=dt, device=dev)
        starts, k = [], 0
        for ps in bucket_params:
            starts.append(k)
            k += len(ps)
        self.fp = FlatParams(model, params=ordered, align=64, shard_multiple=self.world, alloc=alloc,
                             group_starts=starts)
        self.efp = None
        if self.expert_params:
            self.efp = FlatParams(model, params=self.expert_params, align=64)
            self.e_master = self.efp.flat.float()
            self.e_m, self.e_v = torch.zeros_like(self.e_master), torch.zeros_like(self.e_master)
        if self.world > 1:
            dist.broadcast(self.fp.flat, src=dist.get_global_rank(self.group, 0), group=self.group)
        # bucket extents in the flat buffer (each a multiple of 64 * world elements)
        self.bounds = []
        k = 0
        for ps in bucket_params:
            b0 = self.fp.offsets[k]
            k += len(ps)
            b1 = self.fp.offsets[k] if k < len(ordered) else self.fp.total
            self.bounds.append((b0, b1))
        unit = 64 * self.world
        for i, (b0, b1) in enumerate(self.bounds):
            if (b1 - b0) % unit:
                raise RuntimeError("bucket size is not divisible by 64*world; re-pad parameters")
        self.bucket_of_param = {}
        k = 0
        for bi, ps in enumerate(bucket_params):
            for p in ps:
                self.bucket_of_param[id(p)] = bi
        self.bucket_params = bucket_params
        self.shard_total = self.fp.total // self.world
        self.shard_off = [b0 // self.world for (b0, _) in self.bounds]
        # ---- sharded state
        self.master = torch.empty(self.shard_total, dtype=torch.float32, device=dev)
        for bi, (b0, b1) in enumerate(self.bounds):
            sz = (b1 - b0) // self.world
            self.master[self.shard_off[bi]: self.shard_off[bi] + sz].copy_(
                self.fp.flat[b0 + self.rank * sz: b0 + (self.rank + 1) * sz])
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self._nl = len(self.bucket_modules)
        if self.param_slots:
            self._setup_param_slots()
        if self.fused:
            self.pshard = self.sg.alloc(self.shard_total, self.fp.dtype)
            self.pshard.tensor.copy_(self.master)
            self.reduced = torch.empty(self.shard_total, dtype=torch.float32, device=dev)
            self.grid = comm_grid or 2 * torch.cuda.get_device_properties(dev).multi_processor_count
            # one extra slot after the per-bucket partials carries the sum of squares of the local expert gradients
            self.partials = torch.zeros(len(self.bounds) * self.grid + 1, dtype=torch.float32, device=dev)
            self.norm_out = torch.zeros(4, dtype=torch.float32, device=dev)
            if self.nvls and not (self._symm["grad"].multicast_ptr and self._symm["param"].multicast_ptr):
                self.nvls = False          # no multicast mapping on this system: peer loads
            if self.nvls and comm_grid == 0 and os.environ.get("SX_ZERO_NVLS_GRID"):
                self.grid = int(os.environ["SX_ZERO_NVLS_GRID"])
                self.partials = torch.zeros(len(self.bounds) * self.grid + 1, dtype=torch.float32, device=dev)
            self.comm_stream = torch.cuda.Stream(device=dev)
            self.gather_events = [None] * len(self.bounds)
            self._ready_count = 0
            self._status_poll = _lib.StatusPoll(dev)
            self._install_hooks()
            torch.cuda.synchronize()
            dist.barrier(self.group)
        else:
            self.pshard_local = torch.empty(self.shard_total, dtype=self.fp.dtype, device=dev)
            self.pshard_local.copy_(self.master)
            self.reduced = torch.empty(self.shard_total, dtype=torch.float32, device=dev)
            self.gather_events = [None] * len(self.bounds)
            if self.param_slots:
                self._install_hooks()
        self.last_norm = None
        if self.param_slots:
            self._gather_initial()

    # ------------------------------------------------------------------ sharded parameters: rotating layer slots
    def _setup_param_slots(self):
        """Re-homes the parameters: layer i's tensors become views of slot i mod K (at the offsets they had inside
        their bucket), everything outside the layers moves to a compact tail; the full-size buffer is released."""
        K, nl = self.param_slots, self._nl
        assert nl >= K, "fewer layers than parameter slots"
        sizes = {b1 - b0 for (b0, b1) in self.bounds[:nl]}
        rel = [[o - self.bounds[bi][0] for o, p in zip(self.fp.offsets, self.fp.params) if self.bucket_of_param[id(p)] == bi]
               for bi in range(nl)]
        if len(sizes) != 1 or any(r != rel[0] for r in rel):
            raise RuntimeError("param_slots needs identically laid out layers (same parameter shapes in the same order)")
        slot = sizes.pop()
        rest0 = self.bounds[nl][0] if nl < len(self.bounds) else self.fp.total
        old = self.fp.flat
        compact = torch.empty(K * slot + (self.fp.total - rest0), dtype=old.dtype, device=old.device)
        compact[K * slot:].copy_(old[rest0:])
        self._slot_elems, self._rest0, self._compact = slot, rest0, compact
        with torch.no_grad():
            for pr, o in zip(self.fp.params, self.fp.offsets):
                bi = self.bucket_of_param[id(pr)]
                base = (bi % K) * slot + (o - self.bounds[bi][0]) if bi < nl else K * slot + (o - rest0)
                pr.data = compact[base: base + pr.numel()].view(pr.shape)
        self.fp.flat = None          # the only full-size copy of the parameters is gone from here on
        del old
        self._resident = [None] * K  # which layer each slot holds
        self._bwd_events = {}

    def _param_dst(self, bi):
        """Where the gathered parameters of bucket ``bi`` live."""
        b0, b1 = self.bounds[bi]
        if not self.param_slots:
            return self.fp.flat[b0:b1]
        if bi < self._nl:
            k = bi % self.param_slots
            return self._compact[k * self._slot_elems: (k + 1) * self._slot_elems]
        o = self.param_slots * self._slot_elems + (b0 - self._rest0)
        return self._compact[o: o + (b1 - b0)]

    def _gather_bucket(self, bi, after_event=None):
        """All-gather bucket ``bi`` into its destination. Fused path: pull kernel on the comm stream (after
        ``after_event`` of the compute stream, if given), returns the event that marks its end. Library path: a
        blocking ``all_gather`` on the current stream, returns None."""
        b0, b1 = self.bounds[bi]
        sz = (b1 - b0) // self.world
        dst = self._param_dst(bi)
        if bi < self._nl and self.param_slots:
            self._resident[bi % self.param_slots] = bi
        if not self.fused:
            src = self.pshard_local[self.shard_off[bi]: self.shard_off[bi] + sz].contiguous()
            if self.world > 1:
                dist.all_gather_into_tensor(dst, src, group=self.group)
            else:
                dst.copy_(src)
            return None
        cs = self.comm_stream
        if after_event is not None:
            cs.wait_event(after_event)
        es = dst.element_size()
        self.sg.allgather_pull(self.pshard, dst, sz * es, self.shard_off[bi] * es, grid=48,
                               stream=C.c_void_p(cs.cuda_stream))
        ev = torch.cuda.Event()
        ev.record(cs)
        return ev

    def _gather_initial(self):
        """Start of a step with sharded parameters: what runs before the layers, the first K layers, what runs after
        the layers. The compute stream waits for the first group at once, for the others where they are used."""
        nl = self._nl
        self._resident = [None] * self.param_slots      # whatever the slots hold predates the optimizer step
        self._bwd_events = {}
        tail = list(range(nl, len(self.bounds)))
        pre = [b for b in tail if b != self.post_index]
        for bi in pre + list(range(self.param_slots)) + ([self.post_index] if self.post_index is not None else []):
            ev = self._gather_bucket(bi)
            if ev is not None and (bi in pre or not self.bucket_modules):
                torch.cuda.current_stream().wait_event(ev)
            else:
                self.gather_events[bi] = ev

    def _after_layer_forward(self, bi, out):
        """Layer ``bi`` is done with its slot for now: layer ``bi + K`` may be gathered over it; and before the
        backward pass reaches layer ``bi`` its parameters must be back."""
        K, nl = self.param_slots, self._nl
        if bi + K < nl:
            ev = None
            if self.fused:
                ev = torch.cuda.Event()
                ev.record(torch.cuda.current_stream())
            self.gather_events[bi + K] = self._gather_bucket(bi + K, ev)
        if torch.is_grad_enabled():
            outs = out if isinstance(out, (tuple, list)) else (out,)
            for o in outs:
                if torch.is_tensor(o) and o.requires_grad:
                    o.register_hook(lambda g, bi=bi: self._before_layer_backward(bi))
                    break

    def _before_layer_backward(self, bi):
        if self._resident[bi % self.param_slots] != bi:          # library path: gather on demand
            self._gather_bucket(bi)
        ev = self._bwd_events.pop(bi, None)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)

    def _after_layer_backward(self, bi):
        """Layer ``bi``'s backward has been issued: its slot can take layer ``bi - K`` (fused path: ahead of time)."""
        K = self.param_slots
        if self.fused and bi - K >= 0:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            self._bwd_events[bi - K] = self._gather_bucket(bi - K, ev)

    # ------------------------------------------------------------------ fused path plumbing
    def _install_hooks(self):
        eng = self

        def pre_hook_factory(bi):
            def pre(mod, args):
                if eng.param_slots and eng._resident[bi % eng.param_slots] != bi:
                    # not gathered ahead of time (library path; a forward pass outside a training step): do it now
                    e = None
                    if eng.fused:
                        e = torch.cuda.Event()
                        e.record(torch.cuda.current_stream())
                    eng.gather_events[bi] = eng._gather_bucket(bi, e)
                ev = eng.gather_events[bi]
                if ev is not None:
                    torch.cuda.current_stream().wait_event(ev)
                    eng.gather_events[bi] = None
                if torch.is_grad_enabled() and ((eng.fused and eng.stage >= 2) or eng.param_slots):
                    for a in args:
                        if torch.is_tensor(a) and a.requires_grad:
                            a.register_hook(lambda g, bi=bi: eng._layer_backward_done(bi))
                            break
                return None
            return pre

        for bi, mod in enumerate(self.bucket_modules):
            mod.register_forward_pre_hook(pre_hook_factory(bi))
            if self.param_slots:
                mod.register_forward_hook(lambda m_, a_, out, bi=bi: eng._after_layer_forward(bi, out))
        if not self.fused:
            return
        if self.post_index is not None and self.bucket_modules:
            pi = self.post_index

            def after_last_layer(mod, args, out):
                # what follows the layers (final norm, head) needs its gathered parameters now; and its gradients
                # are complete as soon as backward has produced the gradient of this output
                ev = eng.gather_events[pi]
                if ev is not None:
                    torch.cuda.current_stream().wait_event(ev)
                    eng.gather_events[pi] = None
                if torch.is_grad_enabled() and eng.stage >= 2:
                    outs = out if isinstance(out, (tuple, list)) else (out,)
                    for o in outs:
                        if torch.is_tensor(o) and o.requires_grad:
                            o.register_hook(lambda g: eng._bucket_ready(pi))
                            break
                return None

            self.bucket_modules[-1].register_forward_hook(after_last_layer)

    def _launch_reduce(self, bi):
        """Called when bucket ``bi`` holds this rank's complete gradients (stream-ordered on the compute stream)."""
        for p in self.bucket_params[bi]:
            if p.grad is not None:
                if p._main_grad_written:
                    p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                else:
                    p.main_grad.copy_(p.grad)
                p._main_grad_written = True
                p.grad = None
            elif not p._main_grad_written:
                p.main_grad.zero_()
        self._ready_count += 1
        epoch = self._ready_count
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        cs = self.comm_stream
        cs.wait_event(ev)
        sptr = C.c_void_p(cs.cuda_stream)
        self.sg.signal(0, epoch, stream=sptr)
        b0, b1 = self.bounds[bi]
        sz = (b1 - b0) // self.world
        a = self._zero_args()
        a.peers = self.sg.peers(self._symm["grad"])
        a.elem_offset, a.n = b0 + self.rank * sz, sz
        a.reduced = self.reduced.data_ptr() + 4 * self.shard_off[bi]
        a.partial_offset = bi * self.grid
        a.ready_channel, a.ready_epoch = 0, epoch
        a.mode = 1
        if self.nvls:
            a.mc_buf = self._symm["grad"].multicast_ptr
        _lib.call("sx_zero_step", C.byref(a), sptr)

    def _layer_backward_done(self, bi):
        if self.fused and self.stage >= 2:
            self._bucket_ready(bi)
        if self.param_slots:
            self._after_layer_backward(bi)

    def _bucket_ready(self, bi):
        if bi not in self._pending:
            return
        self._pending.discard(bi)
        self._launch_reduce(bi)

    def _zero_args(self):
        from .symm import SxZeroArgs
        a = SxZeroArgs()
        a.sumsq_partials = self.partials.data_ptr()
        a.num_partials = self.partials.numel()
        a.lr, a.beta1, a.beta2, a.eps, a.wd = self.lr, self.betas[0], self.betas[1], self.eps, self.wd
        a.step = self.step_count
        a.max_norm = self.max_grad_norm
        a.grid = self.grid
        a.status = _lib.status_word(self.device).data_ptr()
        return a

    def _prefetch_params(self):
        """Refill the full bf16 parameter buffer from the owners' shards on the comm stream, in forward order:
        what runs before the layers, the layers, what runs after them. Peer-load pull kernels, or (NVLS) one
        multicast store of this rank's shard per bucket."""
        cs = self.comm_stream
        sptr = C.c_void_p(cs.cuda_stream)
        es = self.fp.flat.element_size()
        nl = len(self.bucket_modules)
        tail = list(range(nl, len(self.bounds)))
        pre = [b for b in tail if b != self.post_index]
        order = pre + list(range(nl)) + ([self.post_index] if self.post_index is not None else [])
        for bi in order:
            b0, b1 = self.bounds[bi]
            sz = (b1 - b0) // self.world
            if self.nvls:
                src = self.pshard.tensor[self.shard_off[bi]: self.shard_off[bi] + sz]
                self.sg.allgather_mc(src, self._symm["param"], b0 * es, sz * es, 6, self.sg.next_epoch(6), grid=32,
                                     stream=sptr)
            else:
                self.sg.allgather_pull(self.pshard, self.fp.flat[b0:b1], sz * es, self.shard_off[bi] * es, grid=48,
                                       stream=sptr)
            ev = torch.cuda.Event()
            ev.record(cs)
            if bi in pre or not self.bucket_modules:
                torch.cuda.current_stream().wait_event(ev)   # embeddings: needed first
            else:
                self.gather_events[bi] = ev

    # ------------------------------------------------------------------ step
    def step(self, input_ids, labels, **kw):
        return self._step_fused(input_ids, labels, **kw) if self.fused else self._step_library(input_ids, labels, **kw)

    def _step_fused(self, input_ids, labels, **kw):
        # A bounded device wait that ran out in the previous step left stale gradients / parameters behind:
        # stop here instead of training on them (KernelTimeout; the context stays usable).
        self._status_poll.check()
        self.step_count += 1
        self.fp.begin_step()
        if self.efp is not None:
            self.efp.begin_step()
        self._pending = set(range(len(self.bounds)))
        out = self.model(input_ids, labels=labels, **kw)
        loss = out["loss"] if isinstance(out, dict) else out
        loss.backward()
        # whatever the hooks have not handled (stage 1: everything; otherwise the non-layer bucket), in backward order
        for bi in sorted(self._pending, reverse=True):
            self._launch_reduce(bi)
        self._pending = set()
        cs = self.comm_stream
        if self.efp is not None:
            self.efp.finalize_grads()
            esq, _ = grad_norm_([self.efp.grad])
            self.partials[-1:].copy_(esq[0:1])
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            cs.wait_event(ev)
        sptr = C.c_void_p(cs.cuda_stream)
        a = self._zero_args()
        a.peers = self.sg.peers(self._symm["grad"])
        a.elem_offset, a.n = 0, self.shard_total
        a.reduced = self.reduced.data_ptr()
        a.p32, a.m, a.v = self.master.data_ptr(), self.m.data_ptr(), self.v.data_ptr()
        a.p16_out = self.pshard.tensor.data_ptr()
        a.norm_out = self.norm_out.data_ptr()
        a.norm_channel, a.norm_epoch = 2, self.step_count
        a.done_channel, a.done_epoch = 4, self.step_count
        a.mode = 2
        _lib.call("sx_zero_step", C.byref(a), sptr)
        self.last_norm = self.norm_out
        if self.efp is not None:
            with torch.cuda.stream(cs):   # after the kernel above has produced the clip coefficient
                self._expert_update(self.norm_out[2:3])
            done = torch.cuda.Event()
            done.record(cs)
            torch.cuda.current_stream().wait_event(done)
        if self.param_slots:
            self._gather_initial()
        else:
            self._prefetch_params()
        self._status_poll.arm(cs)
        return loss.detach()

    def check_status(self):
        """Blocking form of the per-step check (e.g. before a checkpoint is written)."""
        if self.fused:
            self._status_poll.check(wait=True)

    def _expert_update(self, coef):
        p16 = self.efp.flat if self.efp.flat.dtype != torch.float32 else None
        target = self.e_master if p16 is not None else self.efp.flat
        adamw_flat_(target, self.e_m, self.e_v, self.efp.grad, p16, self.lr, self.betas[0], self.betas[1], self.eps,
                    self.wd, self.step_count, 1.0, coef)

    def _step_library(self, input_ids, labels, **kw):
        self.step_count += 1
        self.fp.begin_step()
        if self.efp is not None:
            self.efp.begin_step()
        out = self.model(input_ids, labels=labels, **kw)
        loss = out["loss"] if isinstance(out, dict) else out
        loss.backward()
        self.fp.finalize_grads()
        if self.efp is not None:
            self.efp.finalize_grads()
        w, r = self.world, self.rank
        for bi, (b0, b1) in enumerate(self.bounds):
            sz = (b1 - b0) // w
            dst = self.reduced[self.shard_off[bi]: self.shard_off[bi] + sz]
            g = self.fp.grad[b0:b1]
            if dist.get_backend(self.group) == "nccl":
                tmp = torch.empty(sz, dtype=g.dtype, device=g.device)
                dist.reduce_scatter_tensor(tmp, g, group=self.group)
                dst.copy_(tmp)
            else:
                gf = g.float()
                dist.all_reduce(gf, group=self.group)
                dst.copy_(gf[r * sz: (r + 1) * sz])
            dst.div_(w)
        ss = self.reduced.pow(2).sum().reshape(1)
        if self.efp is not None:
            ss = ss + self.efp.grad.float().pow(2).sum().reshape(1)
        dist.all_reduce(ss, group=self.group)
        nrm = ss.sqrt()
        coef = torch.where((nrm > self.max_grad_norm) & (self.max_grad_norm > 0), self.max_grad_norm / (nrm + 1e-6),
                           torch.ones_like(nrm))
        self.last_norm = torch.cat([ss, nrm, coef])
        p16 = self.pshard_local if self.fp.dtype != torch.float32 else None
        adamw_flat_(self.master, self.m, self.v, self.reduced, p16, self.lr, self.betas[0], self.betas[1], self.eps,
                    self.wd, self.step_count, 1.0, coef)
        if self.efp is not None:
            self._expert_update(coef)
        src = self.pshard_local if p16 is not None else self.master
        if p16 is None:
            self.pshard_local.copy_(self.master)
            src = self.pshard_local
        if self.param_slots:
            self._resident = [None] * self.param_slots
            self._gather_initial()
            return loss.detach()
        for bi, (b0, b1) in enumerate(self.bounds):
            sz = (b1 - b0) // w
            dist.all_gather_into_tensor(self.fp.flat[b0:b1], src[self.shard_off[bi]: self.shard_off[bi] + sz].contiguous(),
                                        group=self.group)
        return loss.detach()

    # ------------------------------------------------------------------ sharded state for checkpoints
    def state_dict(self):
        sd = {"step": self.step_count, "master": self.master, "m": self.m, "v": self.v, "rank": self.rank,
              "world": self.world, "bounds": self.bounds}
        if self.efp is not None:
            sd.update(e_master=self.e_master, e_m=self.e_m, e_v=self.e_v)
        return sd

    def load_state_dict(self, sd):
        """Restore this rank's shard and rebuild everything derived from it: the bf16 parameter shard peers gather
        from and the full bf16 parameter buffer the model runs on (gathered from all ranks), so that the first
        step after a resume runs on the restored weights."""
        assert sd["world"] == self.world, "use checkpoint.reshard to change the world size"
        if "rank" in sd and int(sd["rank"]) != self.rank:
            raise ValueError(f"checkpoint shard of rank {int(sd['rank'])} given to rank {self.rank}")
        if "bounds" in sd and [tuple(int(x) for x in b) for b in sd["bounds"]] != [tuple(b) for b in self.bounds]:
            raise ValueError("checkpoint bucket layout differs from this engine's")
        self.step_count = int(sd["step"])
        self.master.copy_(sd["master"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        if self.efp is not None and "e_master" in sd:
            self.e_master.copy_(sd["e_master"])
            self.e_m.copy_(sd["e_m"])
            self.e_v.copy_(sd["e_v"])
            self.efp.flat.copy_(self.e_master)
        self._refresh_params_from_master()

    def _refresh_params_from_master(self):
        w = self.world
        if self.fused:
            self.pshard.tensor.copy_(self.master)
            torch.cuda.synchronize()
            dist.barrier(self.group)          # every rank's shard is in place before anyone pulls
            if self.param_slots:
                self._resident = [None] * self.param_slots
                self._gather_initial()
            else:
                self._prefetch_params()
            self.comm_stream.synchronize()
            torch.cuda.current_stream().wait_stream(self.comm_stream)
            self.gather_events = [None] * len(self.bounds)
            dist.barrier(self.group)
            return
        self.pshard_local.copy_(self.master)
        if self.param_slots:
            self._resident = [None] * self.param_slots
            self._gather_initial()
            return
        for bi, (b0, b1) in enumerate(self.bounds):
            sz = (b1 - b0) // w
            src = self.pshard_local[self.shard_off[bi]: self.shard_off[bi] + sz].contiguous()
            if w > 1:
                dist.all_gather_into_tensor(self.fp.flat[b0:b1], src, group=self.group)
            else:
                self.fp.flat[b0:b1].copy_(src)

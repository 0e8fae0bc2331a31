"""Expert parallelism for the SER MoE layer (F5 / F6).

Experts are split contiguously over the ranks of the EP group (expert e lives on rank e // E_local; the reference
assigns round-robin ``i % ep``, kernel/distributed/expert_parallel.c:53-62 - contiguous blocks keep each owner's
weights one stacked tensor). By default no routed row is ever dropped: the owners' receive buffers (shared by all
layers) hold the worst case, and each layer's activations are sized by the row count of its actual routing, which the
host reads back (4 bytes, behind an event that only waits for the plan kernels) while the shared experts run. Setting
``SX_EP_CAPACITY`` (or ``cap_mult``) switches to capacity-factor routing without the read-back: rows past
``cap_mult`` times the fair share are dropped and counted. Fused path: the routing plan is exchanged through peer stores, the dispatch all-to-all
runs inside the grouped-GEMM kernel (dispatch CTAs push rows into the owners' buffers while GEMM CTAs consume tiles
as their arrival counters fill), and the combine all-to-all is a peer-load gather fused with the top-k weighted
sum. Library path (CPU / ``fused=False``): ``all_to_all_single`` around the local grouped GEMMs.
"""
from __future__ import annotations

import ctypes as C
import os

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import moe as moe_ops
from ..ops.functional import glu
from ..ops.gemm import gemm

CH_PLAN, CH_DISP_SIG, CH_DISP_DONE, CH_COMB_SIG, CH_COMB_DONE = 48, 49, 50, 51, 52


class EPWorkspace:
    """Symmetric buffers of one EP group, shared by all MoE layers (sizes fixed at first use)."""

    def __init__(self, sg, T, k, d, E, cap_mult=None):
        self.sg, self.world, self.rank = sg, sg.world, sg.rank
        self.E, self.E_local = E, E // sg.world
        # No-drop (default): an owner can be sent every routed row of every rank, so its buffers hold world * T * k
        # rows (plus padding of each expert segment to 128). Capacity factor (cap_mult given or SX_EP_CAPACITY set):
        # an owner accepts up to cap_mult times its fair share; rows routed past it are dropped, as in
        # capacity-factor MoE training, and counted in ``dropped``. The reference has no limit because its experts
        # run on the token's own rank (kernel/distributed/expert_parallel.c:70-110).
        if cap_mult is None and os.environ.get("SX_EP_CAPACITY"):
            cap_mult = float(os.environ["SX_EP_CAPACITY"])
        self.cap_mult = cap_mult
        self.nodrop = cap_mult is None
        rows = sg.world * T * k if self.nodrop else min(sg.world * T * k, int(cap_mult * T * k))
        rows += self.E_local * 128
        self.max_rows = (rows + 127) // 128 * 128
        self.max_tiles = self.max_rows // 128
        dev = sg.device
        self.counts_mat = sg.alloc(sg.world * E, torch.int32)
        self.rows_a = sg.alloc(self.max_rows * d, torch.bfloat16)     # forward dispatch target (xs)
        self.rows_b = sg.alloc(self.max_rows * d, torch.bfloat16)     # backward dispatch target (dys)
        self.out = sg.alloc(self.max_rows * d, torch.bfloat16)        # expert outputs read by combine
        self.arrive_a = sg.alloc(self.max_tiles, torch.int32)
        self.arrive_b = sg.alloc(self.max_tiles, torch.int32)
        for b in (self.arrive_a, self.arrive_b, self.counts_mat):
            b.tensor.zero_()
        self.cum_a = torch.zeros(self.max_tiles, dtype=torch.int32, device=dev)
        self.cum_b = torch.zeros(self.max_tiles, dtype=torch.int32, device=dev)
        self.counts = torch.zeros(E, dtype=torch.int32, device=dev)
        self.cta_counter = torch.zeros(8, dtype=torch.int32, device=dev)
        self.dropped = torch.zeros(1, dtype=torch.int32, device=dev)     # routed entries dropped so far (all layers)
        self.d = d
        torch.cuda.synchronize()
        dist.barrier(sg.group)

    def status(self):
        return C.c_void_p(_lib.status_word(self.sg.device).data_ptr())


class EPPlan:
    def __init__(self, ws: EPWorkspace, idx):
        T, k = idx.shape
        dev = idx.device
        self.ws = ws
        self.T, self.k, self.E = T, k, ws.E_local
        self.max_rows, self.max_tiles = ws.max_rows, ws.max_tiles
        i32 = lambda *s: torch.empty(*s, dtype=torch.int32, device=dev)
        self.dest_rank, self.dest_row = i32(T * k), i32(T * k)
        self.tile_group, self.k_ranges = i32(ws.max_tiles), i32(ws.E_local, 2)
        self.expected_a, self.total_rows = i32(ws.max_tiles), i32(1)
        e_base, cursors = i32(ws.E), i32(ws.E)
        prev = ws.cum_a.clone()
        p = ws.sg.peers(ws.counts_mat)
        _lib.call("sx_ep_plan", C.byref(p), _lib.ptr(idx.contiguous()), C.c_longlong(T * k), C.c_int(ws.E),
                  _lib.ptr(ws.counts), C.c_int(CH_PLAN), C.c_uint(ws.sg.next_epoch(CH_PLAN)), _lib.ptr(e_base),
                  _lib.ptr(cursors), _lib.ptr(self.tile_group), _lib.ptr(self.k_ranges), _lib.ptr(ws.cum_a),
                  _lib.ptr(self.expected_a), _lib.ptr(self.total_rows), C.c_int(ws.max_tiles), _lib.ptr(self.dest_rank),
                  _lib.ptr(self.dest_row), _lib.ptr(ws.dropped), ws.status(), _lib.stream())
        self.valid = self.expected_a - prev       # rows that will arrive per tile for this routing
        from ..ops import debug as _dbg
        if _dbg.ENABLED:     # the dispatch pushes rows to (dest_rank, dest_row) of a peer's buffer
            _dbg.check_indices(self.dest_rank, -1, ws.world, _dbg.SITE_EP_RANK)
            _dbg.check_indices(self.dest_row, 0, ws.max_rows, _dbg.SITE_EP_ROW)
            _dbg.check_indices(self.tile_group, -1, ws.E_local, _dbg.SITE_TILE_GROUP)
        self._rows = None if ws.nodrop else ws.max_rows
        if ws.nodrop:
            # rows this rank's experts receive for this routing: read back behind an event that waits for the plan
            # kernels only, so work queued after this point (the shared experts) keeps the GPU busy meanwhile
            self._host = torch.empty(1, dtype=torch.int32).pin_memory()
            self._host.copy_(self.total_rows, non_blocking=True)
            self._event = torch.cuda.Event()
            self._event.record()

    @property
    def rows(self) -> int:
        """Rows (a multiple of 128) of this rank's expert-sorted buffers that this routing uses."""
        if self._rows is None:
            self._event.synchronize()
            self._rows = max(128, min(int(self._host[0]), self.ws.max_rows))
        return self._rows


def _dispatch_gemm(ws, plan, x, w, rows_buf, arrive, expected, scale, b_mn):
    """Push routed rows of ``x`` to their owners and multiply the local expert-sorted rows by ``w`` (one kernel)."""
    d = x.shape[1]
    R = plan.rows
    rows_buf.tensor[: R * d].zero_()
    a_full = rows_buf.tensor[: R * d].view(R, d)
    N = w.shape[2] if b_mn else w.shape[1]
    out = torch.empty(R, N, dtype=x.dtype, device=x.device)
    g = _lib.SxGemmArgs()
    g.A, g.B, g.D = a_full.data_ptr(), w.data_ptr(), out.data_ptr()
    g.M, g.N, g.K, g.batch = R, N, d, 1
    g.lda, g.ldb, g.ldd = d, w.stride(1), N
    g.strideB = w.stride(0)
    g.a_mn, g.b_mn = 0, int(b_mn)
    g.alpha, g.beta = 1.0, 0.0
    g.tile_group, g.num_groups = plan.tile_group.data_ptr(), w.shape[0]
    g.status = _lib.status_word(x.device).data_ptr()
    from .tp import SxGemmCommArgs
    cm = SxGemmCommArgs()
    cm.peers = ws.sg.peers(rows_buf)
    cm.mode = 4
    cm.epoch = ws.sg.next_epoch(CH_DISP_SIG)
    cm.n_copy = 32
    cm.sig_channel, cm.done_channel = CH_DISP_SIG, CH_DISP_DONE
    cm.cta_counter = ws.cta_counter.data_ptr()
    cm.ep_x = x.data_ptr()
    cm.ep_dest_rank, cm.ep_dest_row = plan.dest_rank.data_ptr(), plan.dest_row.data_ptr()
    cm.ep_row_scale = scale.data_ptr() if scale is not None else None
    cm.ep_entries, cm.ep_k, cm.ep_d = plan.T * plan.k, plan.k, d
    for r in range(ws.world):
        cm.ep_arrive[r] = arrive.ptrs[r]
    cm.ep_tile_expected = expected.data_ptr()
    _lib.call("sx_gemm_bf16_comm", C.byref(g), C.byref(cm), _lib.stream())
    return out, a_full


def _combine(ws, plan, w, base, dy, want_y=True, want_dw=False):
    T, k, d = plan.T, plan.k, ws.d
    dev = ws.sg.device
    y = torch.empty(T, d, dtype=torch.bfloat16, device=dev) if want_y else None
    dw = torch.empty(T, k, dtype=torch.float32, device=dev) if want_dw else None
    p = ws.sg.peers(ws.out)
    _lib.call("sx_ep_combine", C.byref(p), _lib.ptr(plan.dest_rank), _lib.ptr(plan.dest_row),
              _lib.ptr(w.contiguous() if w is not None else None), _lib.ptr(base), _lib.ptr(dy), _lib.ptr(y),
              _lib.ptr(dw), C.c_int(T), C.c_int(d), C.c_int(k), C.c_int(CH_COMB_SIG),
              C.c_uint(ws.sg.next_epoch(CH_COMB_SIG)), C.c_int(CH_COMB_DONE),
              C.c_void_p(ws.cta_counter.data_ptr() + 8), ws.status(), _lib.stream())
    return y, dw


class _EPExpertsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, W1, W2, base, ws, plan, act, fp8=False):
        h1, xs_view = _dispatch_gemm(ws, plan, x, W1, ws.rows_a, ws.arrive_a, plan.expected_a, None, False)
        xs = xs_view.clone()
        hm = glu(h1, act)
        out_view = ws.out.tensor[: plan.rows * ws.d].view(plan.rows, ws.d)
        if fp8:       # second expert GEMM in block-scaled e4m3 (the first is fused with the dispatch in bf16)
            from ..ops.quant import gemm_fp8_grouped
            out_view.copy_(gemm_fp8_grouped(hm, plan.tile_group, W2))
        else:
            gemm(hm, W2, tile_group=plan.tile_group, out=out_view)
        y, _ = _combine(ws, plan, w, base, None)
        ctx.save_for_backward(xs, h1, hm, w, W1, W2)
        ctx.ws, ctx.plan, ctx.act, ctx.has_base = ws, plan, act, base is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        xs, h1, hm, w, W1, W2 = ctx.saved_tensors
        ws, plan, act = ctx.ws, ctx.plan, ctx.act
        dy = dy.contiguous()
        # expert outputs again (the shared output buffer has been reused since), for d(gate weights)
        out_view = ws.out.tensor[: plan.rows * ws.d].view(plan.rows, ws.d)
        gemm(hm, W2, tile_group=plan.tile_group, out=out_view)
        _, dw = _combine(ws, plan, None, None, dy, want_y=False, want_dw=True)
        ws.cum_b += plan.valid
        expected_b = ws.cum_b.clone()
        scale = w.detach().reshape(-1).contiguous()
        dhm, dys_view = _dispatch_gemm(ws, plan, dy, W2, ws.rows_b, ws.arrive_b, expected_b, scale, True)
        dW2 = gemm(dys_view, hm, a_mn=True, b_mn=True, k_ranges=plan.k_ranges, out_dtype=torch.float32)
        with torch.enable_grad():
            h1d = h1.detach().requires_grad_(True)
            hm2 = glu(h1d, act)
        (dh1,) = torch.autograd.grad(hm2, h1d, dhm)
        dW1 = gemm(dh1, xs, a_mn=True, b_mn=True, k_ranges=plan.k_ranges, out_dtype=torch.float32)
        gemm(dh1, W1, b_mn=True, tile_group=plan.tile_group, out=out_view)
        dx, _ = _combine(ws, plan, None, None, None)

        def deliver(W, dW):
            mg = getattr(W, "main_grad", None)
            if mg is None:
                return dW.to(W.dtype)
            if getattr(W, "_main_grad_written", False):
                mg.add_(dW.to(mg.dtype))
            else:
                mg.copy_(dW)
            W._main_grad_written = True
            return None

        return dx, dw, deliver(W1, dW1), deliver(W2, dW2), (dy if ctx.has_base else None), None, None, None, None


def _library_forward(layer, x, idx, w, base):
    """all_to_all_single around local grouped GEMMs (baseline; also the CPU/gloo path). Autograd flows through the
    differentiable all-to-all."""
    import torch.distributed.nn.functional as dfn
    group, world, E_local = layer.ep_group, layer.ep_world, layer.E_local
    T, k = idx.shape
    d = x.shape[1]
    flat_e = idx.reshape(-1).long()
    keep = flat_e >= 0
    dest = torch.where(keep, flat_e // E_local, torch.full_like(flat_e, world))
    order = torch.argsort(dest * (layer.E + 1) + flat_e.clamp(min=0), stable=True)
    order = order[keep[order]]
    send_counts = torch.bincount(dest[order], minlength=world)[:world]
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    sc, rc = send_counts.tolist(), recv_counts.tolist()
    tok = order // k
    send_x = x[tok]
    send_e = (flat_e[order] % E_local).to(torch.int64)
    recv_x = dfn.all_to_all_single(torch.empty(sum(rc), d, dtype=x.dtype, device=x.device), send_x, rc, sc, group=group)
    recv_e = torch.empty(sum(rc), dtype=torch.int64, device=x.device)
    dist.all_to_all_single(recv_e, send_e, rc, sc, group=group)
    ones = torch.ones(recv_x.shape[0], 1, dtype=torch.float32, device=x.device)
    ys = moe_ops.experts_forward(recv_x, recv_e.to(torch.int32).view(-1, 1), ones, layer.w1, layer.w2, None, layer.act,
                                 fp8=getattr(layer, "expert_fp8", False))
    back = dfn.all_to_all_single(torch.empty(sum(sc), d, dtype=x.dtype, device=x.device), ys, sc, rc, group=group)
    contrib = back.float() * w.reshape(-1)[order].unsqueeze(1)
    y = torch.zeros(T, d, dtype=torch.float32, device=x.device).index_add(0, tok, contrib)
    if base is not None:
        y = y + base.float()
    return y.to(x.dtype)


_WORKSPACES = {}


def dropped_entries(reset=False) -> int:
    """Routed (token, expert) entries dropped for capacity by this rank's dispatches since start (or last reset)."""
    n = 0
    for ws in _WORKSPACES.values():
        n += int(ws.dropped.item())
        if reset:
            ws.dropped.zero_()
    return n


def policy_name() -> str:
    for ws in _WORKSPACES.values():
        return "no-drop" if ws.nodrop else f"capacity factor {ws.cap_mult}"
    return "no-drop" if not os.environ.get("SX_EP_CAPACITY") else f"capacity factor {os.environ['SX_EP_CAPACITY']}"


def expert_dtype_name(model=None) -> str:
    fp8 = model is not None and any(getattr(m, "expert_fp8", False) for m in model.modules())
    return ("fp8 e4m3 1x128/128x128 forward for the second expert GEMM (the first is fused with the bf16 dispatch), "
            "bf16 backward") if fp8 else "bf16"


FORCE_FUSED = None     # tests set True / False to pin the path of every layer; None: fused for CUDA bf16 tensors


def _use_fused(x, fused):
    if fused is None:
        fused = FORCE_FUSED
    return (x.is_cuda and x.dtype == torch.bfloat16 and _lib.available()) if fused is None else fused


def ep_plan(layer, x, idx, fused=None):
    """Start the routing plan of a fused expert-parallel layer (launches only; returns None on the library path).
    Call it before queueing work that does not depend on the routing (the shared experts), then pass the plan to
    ``ep_experts_forward``."""
    if not _use_fused(x, fused):
        return None
    return EPPlan(_workspace(layer, x, idx), idx)


def _workspace(layer, x, idx):
    ws = getattr(layer, "_ep_ws", None)
    if ws is None:
        from .symm import SymmGroup
        key = (id(layer.ep_group), x.shape[0], idx.shape[1], x.shape[1], layer.E)
        if key not in _WORKSPACES:
            _WORKSPACES[key] = EPWorkspace(SymmGroup(layer.ep_group), x.shape[0], idx.shape[1], x.shape[1], layer.E)
        ws = layer._ep_ws = _WORKSPACES[key]
    return ws


def ep_experts_forward(layer, x, idx, w, base, fused=None, plan=None):
    if not _use_fused(x, fused):
        return _library_forward(layer, x, idx, w, base)
    ws = _workspace(layer, x, idx)
    if plan is None:
        plan = EPPlan(ws, idx)
    return _EPExpertsFn.apply(x, w, layer.w1, layer.w2, base, ws, plan, layer.act, getattr(layer, "expert_fp8", False))

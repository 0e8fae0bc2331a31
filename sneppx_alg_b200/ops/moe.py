"""SER (sparse expert routing) ops: router top-k (M1), routing plan, grouped expert GEMMs (G2) with the
gather / combine kernels around them (the single-GPU halves of F5/F6).

Routing semantics are the reference's (algorithms/ser/core/route.c:94-157): softmax over all experts, top-k with
the lowest index winning ties, renormalised weights; ``aux_losses`` gives its load-balance loss
``E * sum_e f_e * p_e`` (loss.c:31-69) and z-loss ``mean(logit^2)`` (route.c:251-259). ``enforce_capacity`` drops
the lowest-weight assignments of an over-full expert (route.c:290-348).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib
from ._lib import c_int, ptr, stream
from .functional import glu, glu_reference
from .gemm import gemm


def _native(x):
    return x.is_cuda and x.dtype == torch.bfloat16 and _lib.available()


# ----------------------------------------------------------------------------- router
def topk_reference(probs, k):
    """Top-k by probability, ties to the lowest expert index (stable sort)."""
    order = torch.sort(probs, dim=-1, descending=True, stable=True).indices
    return order[:, :k].to(torch.int32)


def route(logits, k, renorm=True):
    """logits [T, E] -> (topk_idx int32 [T,k], topk_w fp32 [T,k] (differentiable), probs fp32 [T,E], counts int32 [E])."""
    T, E = logits.shape
    lf = logits.float()
    probs = torch.softmax(lf, dim=-1)
    if logits.is_cuda and _lib.available() and E <= 256 and k <= 8:
        lc = lf.detach().contiguous()
        idx = torch.empty(T, k, dtype=torch.int32, device=logits.device)
        w_ = torch.empty(T, k, dtype=torch.float32, device=logits.device)
        counts = torch.zeros(E, dtype=torch.int32, device=logits.device)
        parts = _lib.lib().sx_router_parts()
        ps = torch.empty(parts * E, dtype=torch.float32, device=logits.device)
        zs = torch.empty(parts, dtype=torch.float32, device=logits.device)
        _lib.call("sx_router_topk", ptr(lc), ptr(None), ptr(idx), ptr(w_), ptr(counts), ptr(ps), ptr(zs), c_int(T),
                  c_int(E), c_int(k), c_int(int(renorm)), stream())
    else:
        idx = topk_reference(probs.detach(), k)
        counts = torch.bincount(idx.reshape(-1).long(), minlength=E).to(torch.int32)
    w = probs.gather(1, idx.long())          # autograd flows through the (tiny) softmax
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    return idx, w, probs, counts


def aux_losses(logits, probs, counts, k):
    """(load-balance loss, z-loss) of the reference: E * sum_e f_e * p_e with f_e = count_e / T and
    p_e = mean router probability; mean(logit^2)."""
    T, E = probs.shape
    f = counts.float() / max(T, 1)
    p = probs.mean(0)
    return E * (f.detach() * p).sum() / k, logits.float().pow(2).mean()


def enforce_capacity(idx, w, E, capacity):
    """Keep at most ``capacity`` assignments per expert, dropping the lowest weights. Dropped entries get index -1
    and weight 0."""
    T, k = idx.shape
    flat_e = idx.reshape(-1).long()
    flat_w = w.detach().reshape(-1)
    order = torch.argsort(flat_w, descending=True, stable=True)
    e_sorted = flat_e[order]
    onehot = F.one_hot(e_sorted, E)
    rank_in_e = (onehot.cumsum(0) * onehot).sum(-1) - 1
    keep_sorted = rank_in_e < capacity
    keep = torch.zeros_like(keep_sorted)
    keep[order] = keep_sorted
    keep = keep.view(T, k)
    return torch.where(keep, idx, torch.full_like(idx, -1)), w * keep.to(w.dtype)


# ----------------------------------------------------------------------------- routing plan
class MoEPlan:
    """Device-side routing metadata: expert segments padded to 128 rows, tile -> expert table, permutation."""

    def __init__(self, idx, E, all_valid=None):
        """``all_valid``: True when the caller knows that no entry of ``idx`` is -1 (no capacity limit was applied),
        which saves the device -> host read that finding out would cost; None: look."""
        T, k = idx.shape
        dev = idx.device
        self.T, self.k, self.E = T, k, E
        self.max_rows = (T * k + E * 127 + 127) // 128 * 128
        self.max_tiles = self.max_rows // 128
        valid = idx >= 0
        if idx.is_cuda and _lib.available() and (all_valid if all_valid is not None else bool(valid.all())):
            counts = torch.zeros(E, dtype=torch.int32, device=dev)
            counts.scatter_add_(0, idx.reshape(-1).long(), torch.ones(T * k, dtype=torch.int32, device=dev))
            self.offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
            cursors = torch.empty(E, dtype=torch.int32, device=dev)
            self.tile_group = torch.empty(self.max_tiles, dtype=torch.int32, device=dev)
            self.k_ranges = torch.empty(E, 2, dtype=torch.int32, device=dev)
            self.slot = torch.empty(T, k, dtype=torch.int32, device=dev)
            self.row_token = torch.empty(self.max_rows, dtype=torch.int32, device=dev)
            _lib.call("sx_moe_plan", ptr(counts), ptr(idx.contiguous()), ptr(self.offsets), ptr(cursors),
                      ptr(self.tile_group), ptr(self.k_ranges), ptr(self.slot), ptr(self.row_token), c_int(T), c_int(E),
                      c_int(k), c_int(self.max_tiles), stream())
            from . import debug as _dbg
            if _dbg.ENABLED:     # the gather / combine kernels index rows with these
                _dbg.check_indices(idx, 0, E, _dbg.SITE_TILE_GROUP)
                _dbg.check_indices(self.slot, -1, self.max_rows, _dbg.SITE_MOE_SLOT)
                _dbg.check_indices(self.tile_group, -1, E, _dbg.SITE_TILE_GROUP)
        else:
            e = idx.reshape(-1).long()
            ok = e >= 0
            counts = torch.bincount(e[ok], minlength=E)
            padded = (counts + 127) // 128 * 128
            off = torch.zeros(E + 1, dtype=torch.long, device=dev)
            off[1:] = padded.cumsum(0)
            self.offsets = off.to(torch.int32)
            order = torch.argsort(torch.where(ok, e, torch.full_like(e, E)), stable=True)
            rank = torch.empty_like(order)
            sorted_e = torch.where(ok, e, torch.full_like(e, E))[order]
            starts = torch.zeros(E + 2, dtype=torch.long, device=dev)
            starts[1:E + 1] = counts.cumsum(0)
            pos_in_e = torch.arange(e.numel(), device=dev) - starts[sorted_e.clamp(max=E)]
            rank[order] = pos_in_e
            slot = torch.where(ok, off[e.clamp(min=0)] + rank, torch.full_like(e, -1))
            self.slot = slot.view(T, k).to(torch.int32)
            self.row_token = torch.full((self.max_rows,), -1, dtype=torch.int32, device=dev)
            tok = torch.arange(T, device=dev).repeat_interleave(k)
            self.row_token[slot[ok]] = tok[ok].to(torch.int32)
            tiles = torch.arange(self.max_tiles, device=dev) * 128
            tg = torch.searchsorted(off[1:].contiguous(), tiles, right=True)
            self.tile_group = torch.where(tiles < off[E], tg, torch.full_like(tg, -1)).to(torch.int32)
            self.k_ranges = torch.stack([off[:-1], off[1:]], dim=1).to(torch.int32)


def _gather_rows(x, plan):
    if _native(x):
        xs = torch.empty(plan.max_rows, x.shape[1], dtype=x.dtype, device=x.device)
        _lib.call("sx_moe_gather", ptr(x), ptr(plan.row_token), ptr(plan.offsets[plan.E:]), ptr(xs), c_int(x.shape[1]),
                  c_int(plan.max_rows), stream())
        return xs
    rt = plan.row_token.long()
    xs = x[rt.clamp(min=0)] * (rt >= 0).to(x.dtype)[:, None]
    return xs


def _combine(ys, plan, w, base):
    T, d = plan.T, ys.shape[1]
    if _native(ys):
        y = torch.empty(T, d, dtype=ys.dtype, device=ys.device)
        _lib.call("sx_moe_combine", ptr(ys), ptr(plan.slot), ptr(w.contiguous()), ptr(base), ptr(y), c_int(T), c_int(d),
                  c_int(plan.k), stream())
        return y
    s = plan.slot.long()
    g = ys[s.clamp(min=0)].float() * (s >= 0)[..., None] * w[..., None].float()
    y = g.sum(1)
    if base is not None:
        y = y + base.float()
    return y.to(ys.dtype)


def _grouped(a, w, plan, b_mn=False, fp8=False):
    """Row block i of ``a`` times expert tile_group[i]'s matrix. ``fp8``: both operands in block-scaled e4m3
    (1 x 128 activation scales, 128 x 128 weight scales) on the fp8 tensor-core GEMM (forward GEMMs only)."""
    if fp8 and not b_mn:
        from .quant import gemm_fp8_grouped
        return gemm_fp8_grouped(a, plan.tile_group, w)
    if _native(a):
        return gemm(a, w, tile_group=plan.tile_group, b_mn=b_mn)
    out_dim = w.shape[2] if b_mn else w.shape[1]
    out = torch.zeros(a.shape[0], out_dim, dtype=a.dtype, device=a.device)
    off = plan.offsets.tolist()
    for e in range(plan.E):
        if off[e + 1] > off[e]:
            we = w[e].float() if b_mn else w[e].float().t()
            out[off[e]: off[e + 1]] = (a[off[e]: off[e + 1]].float() @ we).to(a.dtype)
    return out


def _grouped_wgrad(dy, x, plan, out_shape, wdtype):
    """dW[e] = dy_e^T x_e over expert e's row segment."""
    if _native(dy):
        return gemm(dy, x, a_mn=True, b_mn=True, k_ranges=plan.k_ranges, out_dtype=torch.float32)
    off = plan.offsets.tolist()
    out = torch.zeros(out_shape, dtype=torch.float32, device=dy.device)
    for e in range(plan.E):
        if off[e + 1] > off[e]:
            out[e] = dy[off[e]: off[e + 1]].float().t() @ x[off[e]: off[e + 1]].float()
    return out


class _ExpertsFn(torch.autograd.Function):
    """y[t] = base[t] + sum_r w[t,r] * Expert_{idx[t,r]}(x[t]) with gated experts W1 [E, 2F, d], W2 [E, d, F]."""

    @staticmethod
    def forward(ctx, x, w, W1, W2, base, plan, act, fp8=False):
        xs = _gather_rows(x, plan)
        h1 = _grouped(xs, W1, plan, fp8=fp8)
        hm = glu(h1, act) if _native(h1) else glu_reference(h1, act)
        ys = _grouped(hm, W2, plan, fp8=fp8)
        y = _combine(ys, plan, w, base)
        ctx.save_for_backward(xs, h1, hm, ys, w, W1, W2)
        ctx.plan, ctx.act, ctx.has_base = plan, act, base is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        xs, h1, hm, ys, w, W1, W2 = ctx.saved_tensors
        plan, act = ctx.plan, ctx.act
        dy = dy.contiguous()
        T, d = dy.shape
        if _native(dy):
            dys = torch.zeros_like(ys)
            dw = torch.empty(T, plan.k, dtype=torch.float32, device=dy.device)
            _lib.call("sx_moe_combine_bwd", ptr(dy), ptr(ys), ptr(plan.slot), ptr(w.contiguous()), ptr(dys), ptr(dw),
                      c_int(T), c_int(d), c_int(plan.k), stream())
        else:
            s = plan.slot.long()
            ok = (s >= 0)
            dw = (ys[s.clamp(min=0)].float() * dy[:, None, :].float()).sum(-1) * ok
            dys = torch.zeros_like(ys)
            contrib = (dy[:, None, :].float() * w[..., None].float()).to(ys.dtype)
            dys[s[ok]] = contrib[ok]
        dhm = _grouped(dys, W2, plan, b_mn=True)
        dW2 = _grouped_wgrad(dys, hm, plan, W2.shape, W2.dtype)
        # gate backward through autograd of the small GLU op
        with torch.enable_grad():
            h1d = h1.detach().requires_grad_(True)
            hm2 = glu(h1d, act) if _native(h1d) else glu_reference(h1d, act)
        (dh1,) = torch.autograd.grad(hm2, h1d, dhm)
        dxs = _grouped(dh1, W1, plan, b_mn=True)
        dW1 = _grouped_wgrad(dh1, xs, plan, W1.shape, W1.dtype)
        if _native(dxs):
            dx = torch.empty(T, d, dtype=dy.dtype, device=dy.device)
            _lib.call("sx_moe_gather_bwd", ptr(dxs), ptr(plan.slot), ptr(dx), c_int(T), c_int(d), c_int(plan.k), stream())
        else:
            s = plan.slot.long()
            dx = (dxs[s.clamp(min=0)].float() * (s >= 0)[..., None]).sum(1).to(dy.dtype)

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

        return dx, dw, deliver(W1, dW1), deliver(W2, dW2), (dy if ctx.has_base else None), None, None, None


def experts_forward(x, idx, w, W1, W2, base=None, act="silu", fp8=False, all_valid=None):
    """x [T, d]; idx int32 [T, k] (-1 = dropped); w fp32 [T, k]; returns [T, d]. ``fp8``: the two forward expert GEMMs
    run in block-scaled e4m3 (the backward GEMMs stay bf16 on the saved bf16 activations: straight-through)."""
    plan = MoEPlan(idx, W1.shape[0], all_valid)
    return _ExpertsFn.apply(x, w, W1, W2, base, plan, act, fp8)


def moe_reference(x, idx, w, W1, W2, base=None, act="silu"):
    """Dense per-token statement of the MoE layer in fp32 (oracle)."""
    T, d = x.shape
    y = torch.zeros(T, d, dtype=torch.float32, device=x.device) if base is None else base.float().clone()
    for r in range(idx.shape[1]):
        for e in range(W1.shape[0]):
            sel = (idx[:, r] == e).nonzero().squeeze(-1)
            if sel.numel() == 0:
                continue
            h = glu_reference((x[sel].float() @ W1[e].float().t()), act)
            y[sel] += w[sel, r, None].float() * (h @ W2[e].float().t())
    return y.to(x.dtype)

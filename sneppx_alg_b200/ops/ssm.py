"""HSS / Mamba-2 state-space ops: causal conv1d (C1) and the chunked SSD scan (S1/S2).

The scan follows the state-space-duality form: per chunk of Q tokens the quadratic term
``(C B^T o L) X`` and the chunk states ``(X o decay)^T B`` are GEMMs (run on the tcgen05 kernel for CUDA
bf16 tensors), chunk boundary states are passed sequentially in fp32, and ``C H`` adds the contribution of
earlier chunks. Backward is the autograd transpose of the same GEMMs. ``ssd_reference`` is the plain
recurrence ``h_t = exp(dt A) h_{t-1} + dt x_t B_t^T ; y_t = C_t h_t + D x_t`` used as the oracle.
The reference's own scan kernels are serial over L (algorithms/hss/cuda/hss_cuda_extended.cu:27-77) and its
Mamba-2 block is a stub (kernel/arch/mamba2.c:36-133); the LTI HSS scan with diagonal A is the special case
of constant dt, B, C.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib
from ._lib import c_int, c_ll, ptr, stream
from .gemm import bmm, gemm


# ----------------------------------------------------------------------------- conv1d (C1)
def conv1d_reference(x, w, bias=None, act=True, prev=None):
    """x [B, L, C], w [C, K] depthwise causal; prev [B, K-1, C] optional left context."""
    B, L, C = x.shape
    K = w.shape[1]
    left = prev if prev is not None else x.new_zeros(B, K - 1, C)
    xp = torch.cat([left, x], dim=1).transpose(1, 2).float()
    y = F.conv1d(xp, w.float().unsqueeze(1), bias.float() if bias is not None else None, groups=C).transpose(1, 2)
    return (F.silu(y) if act else y).to(x.dtype)


class _Conv1dFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, act, prev):
        B, L, C = x.shape
        K = w.shape[1]
        # a column slice of a wider row-major tensor (the xBC part of in_proj's output) is read in place
        if not (x.stride(2) == 1 and x.stride(1) % 8 == 0 and x.stride(1) >= C and x.stride(0) == L * x.stride(1)
                and x.data_ptr() % 16 == 0):
            x = x.contiguous()
        y = torch.empty(B, L, C, dtype=x.dtype, device=x.device)
        _lib.call("sx_conv1d_fwd", ptr(x), ptr(prev), ptr(w), ptr(bias), ptr(y), ptr(None), c_int(B), c_int(L),
                  c_int(C), c_int(K), c_int(int(act)), c_ll(x.stride(1)), stream())
        ctx.save_for_backward(x, w, bias if bias is not None else torch.empty(0), prev if prev is not None else torch.empty(0))
        ctx.meta = (act, bias is not None, prev is not None)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, bias, prev = ctx.saved_tensors
        act, has_b, has_p = ctx.meta
        B, L, C = x.shape
        K = w.shape[1]
        dy = dy.contiguous()
        dx = torch.empty(B, L, C, dtype=x.dtype, device=x.device)
        parts = _lib.lib().sx_conv1d_bwd_parts(c_int(B), c_int(L))
        partial = torch.empty(parts * (K + 1) * C, dtype=torch.float32, device=x.device)
        dwdb = torch.empty((K + 1) * C, dtype=torch.float32, device=x.device)
        _lib.call("sx_conv1d_bwd", ptr(dy), ptr(x), ptr(prev if has_p else None), ptr(w), ptr(bias if has_b else None),
                  ptr(dx), ptr(partial), ptr(dwdb), c_int(B), c_int(L), c_int(C), c_int(K), c_int(int(act)),
                  c_ll(x.stride(1)), stream())
        dw = dwdb[: C * K].view(C, K).to(w.dtype)
        db = dwdb[C * K:].to(w.dtype) if has_b else None
        return dx, dw, db, None, None


def causal_conv1d(x, w, bias=None, act=True, prev=None):
    if x.is_cuda and x.dtype == torch.bfloat16 and _lib.available() and x.shape[-1] % 8 == 0 and w.shape[1] <= 4:
        return _Conv1dFn.apply(x, w, bias, act, prev)
    return conv1d_reference(x, w, bias, act, prev)


class _GateMulFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, z):
        C_ = y.shape[-1]
        rows = y.numel() // C_
        y = y.contiguous()
        zld = z.stride(-2)
        out = torch.empty_like(y)
        _lib.call("sx_gate_mul_fwd", ptr(y), ptr(z), c_ll(zld), ptr(out), c_ll(rows), c_int(C_), stream())
        ctx.save_for_backward(y, z)
        return out

    @staticmethod
    def backward(ctx, g):
        y, z = ctx.saved_tensors
        C_ = y.shape[-1]
        g = g.contiguous()
        dy, dz = torch.empty_like(y), torch.empty(z.shape, dtype=z.dtype, device=z.device)
        _lib.call("sx_gate_mul_bwd", ptr(g), ptr(y), ptr(z), c_ll(z.stride(-2)), ptr(dy), ptr(dz),
                  c_ll(y.numel() // C_), c_int(C_), stream())
        return dy, dz


def gate_mul(y, z):
    """y * silu(z) (the Mamba-2 output gate); z may be a column slice of a wider row-major tensor."""
    C_ = y.shape[-1]
    if (y.is_cuda and y.dtype == torch.bfloat16 and z.dtype == torch.bfloat16 and _lib.available() and C_ % 8 == 0
            and z.shape == y.shape and z.stride(-1) == 1 and z.stride(-2) % 8 == 0 and z.data_ptr() % 16 == 0
            and (z.dim() == 2 or all(z.stride(i) == z.stride(i + 1) * z.shape[i + 1] for i in range(z.dim() - 2)))):
        return _GateMulFn.apply(y, z)
    return (y.float() * F.silu(z.float())).to(y.dtype)


# ----------------------------------------------------------------------------- SSD scan (S1/S2)
def ssd_reference(x, dt, A, Bm, Cm, D=None, init_state=None, return_state=False):
    """Sequential recurrence in fp32. x [B,L,H,P], dt [B,L,H] (>0), A [H] (<0), Bm/Cm [B,L,G,N], D [H]."""
    Bsz, L, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    rep = H // G
    xf, dtf = x.float(), dt.float()
    Bf = Bm.float().repeat_interleave(rep, dim=2)
    Cf = Cm.float().repeat_interleave(rep, dim=2)
    h = torch.zeros(Bsz, H, P, N, dtype=torch.float32, device=x.device) if init_state is None else init_state.float()
    ys = []
    for t in range(L):
        dA = torch.exp(dtf[:, t] * A.float())                      # [B,H]
        h = h * dA[..., None, None] + (dtf[:, t, :, None] * xf[:, t])[..., None] * Bf[:, t, :, None, :]
        ys.append(torch.einsum("bhpn,bhn->bhp", h, Cf[:, t]))
    y = torch.stack(ys, dim=1)
    if D is not None:
        y = y + xf * D.float().view(1, 1, H, 1)
    y = y.to(x.dtype)
    return (y, h) if return_state else y


def ssd_chunked(x, dt, A, Bm, Cm, D=None, chunk=64, init_state=None, return_state=False):
    """Chunked SSD with GEMM-shaped work. Same arguments as ``ssd_reference``; L is padded to a multiple of chunk."""
    Bsz, L, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    rep = H // G
    Q = chunk
    pad = (-L) % Q
    if pad:
        x = F.pad(x, (0, 0, 0, 0, 0, pad))
        dt = F.pad(dt, (0, 0, 0, pad))
        Bm = F.pad(Bm, (0, 0, 0, 0, 0, pad))
        Cm = F.pad(Cm, (0, 0, 0, 0, 0, pad))
    Lp = L + pad
    nc = Lp // Q
    cdt = x.dtype
    dA = (dt.float() * A.float()).view(Bsz, nc, Q, H)                      # [B,nc,Q,H]
    cs = torch.cumsum(dA, dim=2)                                           # inclusive
    dtc = dt.float().view(Bsz, nc, Q, H)
    xc = x.view(Bsz, nc, Q, H, P)
    Bc = Bm.view(Bsz, nc, Q, G, N).permute(0, 1, 3, 2, 4)                  # [B,nc,G,Q,N]
    Cc = Cm.view(Bsz, nc, Q, G, N).permute(0, 1, 3, 2, 4)
    # 1. intra-chunk: (C B^T o L o dt) X
    CB = bmm(Cc.contiguous(), Bc.transpose(-1, -2).contiguous())           # [B,nc,G,Q,Q]
    csh = cs.permute(0, 1, 3, 2)                                           # [B,nc,H,Q]
    seg = csh[..., :, None] - csh[..., None, :]                            # l - s
    mask = torch.ones(Q, Q, dtype=torch.bool, device=x.device).tril()
    Lmat = torch.exp(seg.masked_fill(~mask, float("-inf")))                # [B,nc,H,Q,Q]
    M = (CB.float().repeat_interleave(rep, dim=2) * Lmat * dtc.permute(0, 1, 3, 2)[..., None, :]).to(cdt)
    xh = xc.permute(0, 1, 3, 2, 4).contiguous()                            # [B,nc,H,Q,P]
    Y = bmm(M, xh).float()                                                 # [B,nc,H,Q,P]
    # 2. chunk states: S[c] = sum_s exp(cs_last - cs_s) dt_s x_s B_s^T -> [B,nc,H,P,N]
    decay = torch.exp(csh[..., -1:] - csh) * dtc.permute(0, 1, 3, 2)       # [B,nc,H,Q]
    xw = (xh.float() * decay[..., None]).to(cdt)                           # [B,nc,H,Q,P]
    Bh = Bc.repeat_interleave(rep, dim=2).contiguous()                     # [B,nc,H,Q,N]
    S = bmm(xw.transpose(-1, -2).contiguous(), Bh).float()                 # [B,nc,H,P,N]
    # 3. pass states across chunks (fp32, sequential over nc)
    tot = torch.exp(csh[..., -1])                                          # [B,nc,H]
    h = torch.zeros(Bsz, H, P, N, dtype=torch.float32, device=x.device) if init_state is None else init_state.float()
    prev_states = []
    for c in range(nc):
        prev_states.append(h)
        h = h * tot[:, c, :, None, None] + S[:, c]
    Hprev = torch.stack(prev_states, dim=1)                                # [B,nc,H,P,N] state entering each chunk
    # 4. inter-chunk: exp(cs) * C H^T
    Ch = Cc.repeat_interleave(rep, dim=2).contiguous()                     # [B,nc,H,Q,N]
    Yoff = bmm(Ch, Hprev.to(cdt).transpose(-1, -2).contiguous()).float()   # [B,nc,H,Q,P]
    Y = Y + Yoff * torch.exp(csh)[..., None]
    y = Y.permute(0, 1, 3, 2, 4).reshape(Bsz, Lp, H, P)
    if D is not None:
        y = y + x.float() * D.float().view(1, 1, H, 1)
    y = y[:, :L].to(cdt)
    return (y, h) if return_state else y


# ---- building blocks of the chunked scan; each has a CUDA kernel and the plain PyTorch statement below it
def _mask(Q, dev):
    return torch.ones(Q, Q, dtype=torch.bool, device=dev).tril()


def _build_m(CB, csh, dth, rep, cdt):
    """M[l,s] = CB[l,s] exp(cs_l - cs_s) dt_s for s <= l (else 0). CB [B,nc,G,Q,Q] fp32; csh, dth [B,nc,H,Q] fp32."""
    Bsz, nc, G, Q, _ = CB.shape
    H = csh.shape[2]
    if CB.is_cuda and cdt == torch.bfloat16 and _lib.available():
        M = torch.empty(Bsz, nc, H, Q, Q, dtype=cdt, device=CB.device)
        _lib.call("sx_ssd_build_m", ptr(CB), ptr(csh), ptr(dth), ptr(M), c_ll(Bsz * nc), c_int(H), c_int(G), c_int(Q),
                  stream())
        return M
    seg = csh[..., :, None] - csh[..., None, :]
    Lm = torch.exp(seg.masked_fill(~_mask(Q, CB.device), float("-inf"))) * dth[..., None, :]
    return (CB.repeat_interleave(rep, dim=2) * Lm).to(cdt)


def _bwd_qq(dM, CB, csh, dth, rep, cdt):
    """From dM = dY X^T per head: M (as in ``_build_m``), dGh = dM o L o dt, rowW[l] = sum_s dM M,
    colU[s] = sum_l dM CB L (so that sum_l dM M = colU dt_s without a division by dt)."""
    Bsz, nc, G, Q, _ = CB.shape
    H = csh.shape[2]
    if CB.is_cuda and cdt == torch.bfloat16 and _lib.available():
        M = torch.empty(Bsz, nc, H, Q, Q, dtype=cdt, device=CB.device)
        dGh = torch.empty_like(M)
        rowW = torch.empty(Bsz, nc, H, Q, dtype=torch.float32, device=CB.device)
        colU = torch.empty_like(rowW)
        _lib.call("sx_ssd_bwd_qq", ptr(dM), ptr(CB), ptr(csh), ptr(dth), ptr(M), ptr(dGh), ptr(rowW), ptr(colU),
                  c_ll(Bsz * nc), c_int(H), c_int(G), c_int(Q), stream())
        return M, dGh, rowW, colU
    seg = csh[..., :, None] - csh[..., None, :]
    Lexp = torch.exp(seg.masked_fill(~_mask(Q, CB.device), float("-inf")))
    CBh = CB.repeat_interleave(rep, dim=2)
    dMf = dM.float().view(Bsz, nc, H, Q, Q)
    Lm = Lexp * dth[..., None, :]
    U = dMf * CBh * Lexp
    return (CBh * Lm).to(cdt), (dMf * Lm).to(cdt), (U * dth[..., None, :]).sum(-1), U.sum(-2)


def _state_fwd(S, tot, init, cdt):
    """H_0 = init; H_{c+1} = tot_c H_c + S_c. Returns the state entering every chunk (cdt) and the final state (fp32)."""
    Bsz, nc, H, P, N = S.shape
    if S.is_cuda and cdt == torch.bfloat16 and _lib.available() and (P * N) % 8 == 0:
        Hprev = torch.empty(Bsz, nc, H, P, N, dtype=cdt, device=S.device)
        final = torch.empty(Bsz, H, P, N, dtype=torch.float32, device=S.device)
        init32 = init.float().contiguous() if init is not None else None
        _lib.call("sx_ssd_state_fwd", ptr(S), ptr(tot), ptr(init32), ptr(Hprev), ptr(final), c_int(Bsz), c_int(nc),
                  c_int(H), c_int(P * N), stream())
        return Hprev, final
    h = torch.zeros(Bsz, H, P, N, dtype=torch.float32, device=S.device) if init is None else init.float()
    prev = []
    for c in range(nc):
        prev.append(h.to(cdt))
        h = h * tot[:, c, :, None, None] + S[:, c]
    return torch.stack(prev, dim=1), h


def _state_bwd(dHprev, tot, Hprev, dfinal):
    """Reverse of ``_state_fwd``: dS_c = dH_{c+1}; dtot_c = <dH_{c+1}, H_c>; dH_c = tot_c dH_{c+1} + dHprev_c."""
    Bsz, nc, H, P, N = dHprev.shape
    if dHprev.is_cuda and Hprev.dtype == torch.bfloat16 and _lib.available() and (P * N) % 8 == 0:
        dS = torch.empty(Bsz, nc, H, P, N, dtype=torch.bfloat16, device=dHprev.device)
        dtot = torch.zeros(Bsz, nc, H, dtype=torch.float32, device=dHprev.device)
        dinit = torch.empty(Bsz, H, P, N, dtype=torch.float32, device=dHprev.device)
        df = dfinal.float().contiguous() if dfinal is not None else None
        _lib.call("sx_ssd_state_bwd", ptr(dHprev), ptr(tot), ptr(Hprev), ptr(df), ptr(dS), ptr(dtot), ptr(dinit),
                  c_int(Bsz), c_int(nc), c_int(H), c_int(P * N), stream())
        return dS, dtot, dinit
    run = torch.zeros(Bsz, H, P, N, dtype=torch.float32, device=dHprev.device) if dfinal is None else dfinal.float()
    dS, dtot = [None] * nc, [None] * nc
    for c in range(nc - 1, -1, -1):
        dS[c] = run
        dtot[c] = (run * Hprev[:, c].float()).sum((-1, -2))
        run = run * tot[:, c, :, None, None] + dHprev[:, c]
    return torch.stack(dS, dim=1).to(Hprev.dtype), torch.stack(dtot, dim=1), run


def _to_gf(t5, G):
    """Token-major [B,nc,Q,H,P] -> group-first [B*nc*G, Q, (H/G)*P] (a view of the same memory for G == 1)."""
    B_, nc, Q, H, P = t5.shape
    if G == 1:
        return t5.reshape(B_ * nc, Q, H * P)
    return t5.reshape(B_, nc, Q, G, (H // G) * P).permute(0, 1, 3, 2, 4).reshape(B_ * nc * G, Q, (H // G) * P)


def _from_gf(t3, shape5, G):
    """Inverse of ``_to_gf``."""
    B_, nc, Q, H, P = shape5
    if G == 1:
        return t3.reshape(shape5)
    return t3.reshape(B_, nc, G, Q, (H // G) * P).permute(0, 1, 3, 2, 4).reshape(shape5)


def _scale_rows(t5, scale, cdt, G):
    """t5 [B,nc,Q,H,P] times scale [B,nc,Q,H] (fp32), rounded to the compute dtype, in group-first layout."""
    B_, nc, Q, H, P = t5.shape
    if t5.is_cuda and t5.dtype == torch.bfloat16 and cdt == torch.bfloat16 and _lib.available() and P % 8 == 0:
        out = torch.empty(B_ * nc * G, Q, (H // G) * P, dtype=cdt, device=t5.device)
        _lib.call("sx_ssd_scale_rows", ptr(t5), ptr(scale.contiguous()), ptr(out), c_ll(scale.numel()),
                  c_int(P), c_int(H), c_ll(t5.stride(2)), c_int(Q), c_int(G), stream())
        return out
    return _to_gf((t5.float() * scale[..., None]).to(cdt), G)


def _rows_kernel_ok(t5, cdt):
    P = t5.shape[-1]
    return (t5.is_cuda and cdt == torch.bfloat16 and t5.dtype == torch.bfloat16 and _lib.available() and P % 8 == 0
            and (P // 8) & (P // 8 - 1) == 0 and P <= 256)


def _combine(Yi, Yoff, x5, E, D, cdt, G):
    """y = Yi (heads-first [B,nc,H,Q,P]) + E Yoff (group-first) + D x on the token-major layout [B,nc,Q,H,P]."""
    B_, nc, Q, H, P = x5.shape
    if _rows_kernel_ok(x5, cdt):
        y = torch.empty(x5.shape, dtype=cdt, device=x5.device)
        _lib.call("sx_ssd_combine", ptr(Yi), ptr(Yoff), ptr(x5), ptr(E), ptr(D.float().contiguous() if D is not None else None),
                  ptr(y), c_ll(B_ * nc * Q * H), c_int(H), c_int(Q), c_int(P), c_ll(x5.stride(2)), c_int(G), stream())
        return y
    y = Yi.float().permute(0, 1, 3, 2, 4) + _from_gf(Yoff, x5.shape, G).float() * E[..., None]
    if D is not None:
        y = y + x5.float() * D.float().view(H, 1)
    return y.to(cdt)


def _bwd_rows1(dy5, x5, Yoff, E, cdt, G):
    """dye = dy E (compute dtype, group-first); dcs = sum_p dy E Yoff; ddrow = sum_p dy x. Yoff is group-first."""
    if _rows_kernel_ok(x5, cdt) and dy5.dtype == cdt:
        dye = torch.empty_like(Yoff)
        dcs = torch.empty(E.shape, dtype=torch.float32, device=E.device)
        ddrow = torch.empty_like(dcs)
        _lib.call("sx_ssd_bwd_rows1", ptr(dy5), ptr(x5), ptr(Yoff), ptr(E), ptr(dye), ptr(dcs), ptr(ddrow),
                  c_ll(E.numel()), c_int(x5.shape[-1]), c_int(x5.shape[-2]), c_ll(x5.stride(2)), c_int(x5.shape[2]),
                  c_int(G), stream())
        return dye, dcs, ddrow
    dyf = dy5.float()
    dyeE = dyf * E[..., None]
    return (_to_gf(dyeE.to(cdt), G), (dyeE * _from_gf(Yoff, x5.shape, G).float()).sum(-1),
            (dyf * x5.float()).sum(-1))


def _bwd_rows2(dy5, x5, dxw, dxi, decay, D, cdt, G):
    """dx = D dy + decay dxw (group-first) + dxi (heads-first [B,nc,H,Q,P]); ddecay = sum_p dxw x."""
    B_, nc, Q, H, P = x5.shape
    if _rows_kernel_ok(x5, cdt) and dy5.dtype == cdt:
        dx = torch.empty(x5.shape, dtype=cdt, device=x5.device)
        ddecay = torch.empty(decay.shape, dtype=torch.float32, device=decay.device)
        _lib.call("sx_ssd_bwd_rows2", ptr(dy5), ptr(x5), ptr(dxw), ptr(dxi), ptr(decay),
                  ptr(D.float().contiguous() if D is not None else None), ptr(dx), ptr(ddecay), c_ll(decay.numel()),
                  c_int(H), c_int(Q), c_int(P), c_ll(x5.stride(2)), c_int(G), stream())
        return dx, ddecay
    dxw5 = _from_gf(dxw, x5.shape, G).float()
    dx = dxw5 * decay[..., None] + dxi.float().permute(0, 1, 3, 2, 4)
    if D is not None:
        dx = dx + dy5.float() * D.float().view(H, 1)
    return dx.to(cdt), (dxw5 * x5.float()).sum(-1)


class _Chunks:
    """Shapes, padded chunk views and the per-chunk cumulative decay shared by forward and backward."""

    def __init__(self, x, dt, A, Bm, Cm, Q):
        self.Bsz, self.L, self.H, self.P = x.shape
        self.G, self.N = Bm.shape[2], Bm.shape[3]
        self.rep = self.H // self.G
        self.Q = Q
        self.pad = (-self.L) % Q
        if self.pad:
            x = F.pad(x, (0, 0, 0, 0, 0, self.pad))
            dt = F.pad(dt, (0, 0, 0, self.pad))
            Bm = F.pad(Bm, (0, 0, 0, 0, 0, self.pad))
            Cm = F.pad(Cm, (0, 0, 0, 0, 0, self.pad))
        self.Lp = self.L + self.pad
        self.nc = nc = self.Lp // Q
        B_, H, P, G, N = self.Bsz, self.H, self.P, self.G, self.N
        self.cdt = x.dtype
        # token-major ("natural") layout; a column slice of a wider row-major tensor (x inside the conv output)
        # is used in place: the kernels take the token stride
        if not (x.is_cuda and x.stride(3) == 1 and x.stride(2) == P and x.stride(0) == self.Lp * x.stride(1)
                and x.stride(1) % 8 == 0 and x.data_ptr() % 16 == 0):
            x = x.contiguous()
        self.x5 = x.view(B_, nc, Q, H, P)
        self.dtf = dt.float().reshape(B_, nc, Q, H)
        self.dth = self.dtf.permute(0, 1, 3, 2).contiguous()                     # [B,nc,H,Q]
        self.csh = torch.cumsum(self.dth * A.float().view(H, 1), dim=-1)         # inclusive, along the chunk
        self.cs = self.csh.permute(0, 1, 3, 2).contiguous()                      # [B,nc,Q,H]
        self.Bc = Bm.to(self.cdt).reshape(B_, nc, Q, G, N).permute(0, 1, 3, 2, 4).contiguous().view(B_ * nc, G, Q, N)
        self.Cc = Cm.to(self.cdt).reshape(B_, nc, Q, G, N).permute(0, 1, 3, 2, 4).contiguous().view(B_ * nc, G, Q, N)
        self._CB = None
        self.eL = torch.exp(self.cs[:, :, -1:, :] - self.cs)                     # exp(cs_last - cs_s)
        self.decay = self.eL * self.dtf
        self.tot = torch.exp(self.cs[:, :, -1, :]).contiguous()                  # [B,nc,H]
        self.xw = _scale_rows(self.x5, self.decay, self.cdt, G)               # group-first [B*nc*G, Q, rep*P]

    @property
    def CB(self):
        """C B^T per (chunk, group), fp32 [B,nc,G,Q,Q] (built on first use: the fused forward kernel keeps it in TMEM)."""
        if self._CB is None:
            Q, N = self.Q, self.N
            self._CB = gemm(self.Cc.view(-1, Q, N), self.Bc.view(-1, Q, N), out_dtype=torch.float32).view(
                self.Bsz, self.nc, self.G, Q, Q)
        return self._CB

    def by_group(self, t):
        """[.., H*P, N] states or [B*nc, G, Q, N] projections as one batch of (chunk, group) matrices."""
        return t.reshape(self.Bsz * self.nc * self.G, -1, self.N)

    def heads_first(self, t5):
        """[B,nc,Q,H,P] -> contiguous [B*nc*H, Q, P]."""
        if t5.is_cuda and t5.dtype == torch.bfloat16 and _lib.available() and self.P % 8 == 0:
            out = torch.empty(self.Bsz * self.nc * self.H, self.Q, self.P, dtype=t5.dtype, device=t5.device)
            _lib.call("sx_ssd_heads_first", ptr(t5), c_ll(t5.stride(2)), ptr(out), c_ll(out.shape[0] * self.Q),
                      c_int(self.H), c_int(self.Q), c_int(self.P), stream())
            return out
        return t5.permute(0, 1, 3, 2, 4).contiguous().view(-1, self.Q, self.P)

    def y_off(self, Hprev):
        B_, nc, Q, H, P, N = self.Bsz, self.nc, self.Q, self.H, self.P, self.N
        return gemm(self.by_group(self.Cc), self.by_group(Hprev))              # group-first [B*nc*G, Q, rep*P]


def _token_major_ok(t, inner):
    """[B, L, G, inner] readable in place by TMA: unit inner stride, dense (G, inner), batch stride = L * token stride."""
    return (t.stride(3) == 1 and t.stride(2) == inner and t.stride(0) == t.shape[1] * t.stride(1)
            and t.stride(1) % 8 == 0 and t.data_ptr() % 16 == 0)


def _chunk_fwd_fused(k, Bm, Cm, D, Hprev):
    """Output stage of the scan in one tcgen05 kernel (csrc/ssd_fwd.cu): C B^T stays in TMEM across the heads of a
    group, M = C B^T o L o dt goes to the M X product straight from TMEM and the C Hprev^T term, the exp(cs) scaling
    and D x are applied in its epilogue. Covers chunk 128, state 128, headdim 64 without padding; returns None
    otherwise (``SX_SSD_FUSED=0`` forces the staged path)."""
    import os
    if not (k.x5.is_cuda and k.cdt == torch.bfloat16 and k.Q == 128 and k.N == 128 and k.P == 64 and k.pad == 0
            and _lib.available() and k.Bsz * k.nc <= 65535 and os.environ.get("SX_SSD_FUSED", "1") != "0"
            and Bm.dtype == torch.bfloat16 and Cm.dtype == torch.bfloat16):
        return None
    if not _token_major_ok(Bm, k.N):
        Bm = Bm.contiguous()
    if not _token_major_ok(Cm, k.N):
        Cm = Cm.contiguous()
    y = torch.empty(k.Bsz, k.nc, k.Q, k.H, k.P, dtype=k.cdt, device=k.x5.device)
    Dp = D.float().contiguous() if D is not None else None
    _lib.call("sx_ssd_chunk_fwd", ptr(Cm), c_ll(Cm.stride(1)), ptr(Bm), c_ll(Bm.stride(1)), ptr(k.x5),
              c_ll(k.x5.stride(2)), ptr(Hprev), ptr(k.csh), ptr(k.dth), ptr(Dp), ptr(y), c_ll(k.Bsz * k.nc),
              c_int(k.H), c_int(k.G), _lib.c_void_p(_lib.status_word(k.x5.device).data_ptr()), stream())
    return y


class _SSDFn(torch.autograd.Function):
    """Chunked SSD scan with a hand-written backward. Only the inputs and the chunk-entry states are kept for
    backward; every Q x Q quantity is rebuilt there, so the memory held per layer is O(L) rather than O(L Q)."""

    @staticmethod
    def forward(ctx, x, dt, A, Bm, Cm, D, init_state, chunk):
        ctx.set_materialize_grads(False)
        k = _Chunks(x, dt, A, Bm, Cm, chunk)
        B_, nc, Q, H, P, N = k.Bsz, k.nc, k.Q, k.H, k.P, k.N
        S = gemm(k.xw, k.by_group(k.Bc), a_mn=True, b_mn=True, out_dtype=torch.float32)   # [B*nc*G, rep*P, N]
        Hprev, final = _state_fwd(S.view(B_, nc, H, P, N), k.tot, init_state, k.cdt)
        y = _chunk_fwd_fused(k, Bm, Cm, D, Hprev)
        if y is None:
            M = _build_m(k.CB, k.csh, k.dth, k.rep, k.cdt)
            Yi = gemm(M.view(-1, Q, Q), k.heads_first(k.x5), b_mn=True).view(B_, nc, H, Q, P)
            y = _combine(Yi, k.y_off(Hprev), k.x5, torch.exp(k.cs), D, k.cdt, k.G)
        ctx.save_for_backward(x, dt, A, Bm, Cm, D, Hprev)
        ctx.chunk = chunk
        ctx.has_init = init_state is not None
        return y.reshape(B_, k.Lp, H, P)[:, :k.L], final

    @staticmethod
    def backward(ctx, dy, dfinal):
        x, dt, A, Bm, Cm, D, Hprev = ctx.saved_tensors
        k = _Chunks(x, dt, A, Bm, Cm, ctx.chunk)
        B_, nc, Q, H, P, N, G = k.Bsz, k.nc, k.Q, k.H, k.P, k.N, k.G
        dev, cdt = x.device, k.cdt
        if dy is None:
            dy = torch.zeros_like(x)
        if k.pad:
            dy = F.pad(dy, (0, 0, 0, 0, 0, k.pad))
        dy5 = dy.to(cdt).contiguous().view(B_, nc, Q, H, P)
        # ---- contribution of earlier chunks: y_off = exp(cs) C H_prev^T
        dye, dcs, ddrow = _bwd_rows1(dy5, k.x5, k.y_off(Hprev), torch.exp(k.cs), cdt, G)
        dD = ddrow.sum((0, 1, 2)) if D is not None else None
        Hp, Cg, Bg = k.by_group(Hprev), k.by_group(k.Cc), k.by_group(k.Bc)
        dC = gemm(dye, Hp, b_mn=True, out_dtype=torch.float32).view(B_ * nc, G, Q, N)
        dHprev = gemm(dye, Cg, a_mn=True, b_mn=True, out_dtype=torch.float32)     # [B*nc*G, rep*P, N]
        # ---- chunk-to-chunk recurrence, reversed
        dS, dtot, dinit = _state_bwd(dHprev.view(B_, nc, H, P, N), k.tot, Hprev, dfinal)
        dcs_last = dtot * k.tot                                                  # [B,nc,H]
        # ---- chunk states S = (x o decay)^T B
        dSb = k.by_group(dS)
        dxw = gemm(Bg, dSb)                                                      # group-first [B*nc*G, Q, rep*P]
        dB = gemm(k.xw, dSb, b_mn=True, out_dtype=torch.float32).view(B_ * nc, G, Q, N)
        # ---- quadratic term within the chunk
        dyh = k.heads_first(dy5)
        xh = k.heads_first(k.x5)
        dM = gemm(dyh, xh)                                                       # [n,Q,Q]
        M, dGh, rowW, colU = _bwd_qq(dM.view(B_, nc, H, Q, Q), k.CB, k.csh, k.dth, k.rep, cdt)
        dxi = gemm(M.view(-1, Q, Q), dyh, a_mn=True, b_mn=True).view(B_, nc, H, Q, P)
        dx, ddecay = _bwd_rows2(dy5, k.x5, dxw, dxi, k.decay, D, cdt, G)
        gdec = ddecay * k.decay
        dcs_last = dcs_last + gdec.sum(2)
        dcs = dcs - gdec + (rowW - colU * k.dth).permute(0, 1, 3, 2)
        ddt = ddecay * k.eL + colU.permute(0, 1, 3, 2)
        dG = dGh.view(B_ * nc, G, k.rep, Q, Q)
        dG = (dG.sum(2, dtype=torch.float32).to(cdt) if k.rep > 1 else dG[:, :, 0]).reshape(-1, Q, Q)
        dC += gemm(dG, k.Bc.view(-1, Q, N), b_mn=True, out_dtype=torch.float32).view(B_ * nc, G, Q, N)
        dB += gemm(dG, k.Cc.view(-1, Q, N), a_mn=True, b_mn=True, out_dtype=torch.float32).view(B_ * nc, G, Q, N)
        # ---- cs = cumsum(dt A) within the chunk
        dcs[:, :, -1, :] += dcs_last
        dch = dcs.permute(0, 1, 3, 2).contiguous()                               # reverse cumulative sum along the chunk
        da = (dch.sum(-1, keepdim=True) - torch.cumsum(dch, -1) + dch).permute(0, 1, 3, 2)
        ddt += da * A.float()
        dA = (da * k.dtf).sum((0, 1, 2))
        L = k.L
        tok = lambda t: t.view(B_, nc, G, Q, N).permute(0, 1, 3, 2, 4).reshape(B_, k.Lp, G, N)[:, :L]
        return (dx.reshape(B_, k.Lp, H, P)[:, :L].to(x.dtype), ddt.reshape(B_, k.Lp, H)[:, :L].to(dt.dtype),
                dA.to(A.dtype), tok(dB).to(Bm.dtype), tok(dC).to(Cm.dtype),
                dD.to(D.dtype) if D is not None else None, dinit if ctx.has_init else None, None)


def ssd_scan(x, dt, A, Bm, Cm, D=None, chunk=64, init_state=None, return_state=False):
    """Chunked SSD scan (forward and backward hand-written; see ``_SSDFn``). Same arguments as ``ssd_reference``."""
    L = x.shape[1]
    chunk = max(8, min(int(chunk), 256))
    if chunk & (chunk - 1):
        chunk = 1 << (chunk.bit_length() - 1)          # the Q x Q kernels take power-of-two chunks
    while chunk > 8 and chunk // 2 >= L:
        chunk //= 2
    y, final = _SSDFn.apply(x, dt, A, Bm, Cm, D, init_state, chunk)
    return (y, final) if return_state else y


def ssd_step(h, x, dt, A, Bm, Cm, D=None):
    """Single-token recurrence for decoding. h [B,H,P,N]; x [B,H,P]; dt [B,H]; Bm/Cm [B,G,N]."""
    H, G = x.shape[1], Bm.shape[1]
    rep = H // G
    Bf = Bm.float().repeat_interleave(rep, dim=1)
    Cf = Cm.float().repeat_interleave(rep, dim=1)
    dA = torch.exp(dt.float() * A.float())
    h = h * dA[..., None, None] + (dt.float()[..., None] * x.float())[..., None] * Bf[:, :, None, :]
    y = torch.einsum("bhpn,bhn->bhp", h, Cf)
    if D is not None:
        y = y + x.float() * D.float().view(1, H, 1)
    return y.to(x.dtype), h

"""Autograd front-ends of the sm_100a kernels, each paired with a plain PyTorch statement of the
same math (``*_reference``) that serves CPU tensors and is the oracle the GPU tests compare with.

CUDA bf16 tensors always take the native kernel; if the library cannot be loaded on a machine
with a GPU the call raises instead of silently running PyTorch kernels.
"""
from __future__ import annotations

import ctypes as C
import math

import torch
import torch.nn.functional as F

from . import _lib
from ._lib import c_float, c_int, c_ll, ptr, stream
from .gemm import gemm, linear  # noqa: F401  (re-exported)


def _native(*ts) -> bool:
    t = ts[0]
    return t.is_cuda and t.dtype == torch.bfloat16 and _lib.available()


# ----------------------------------------------------------------------------- RMSNorm (N1)
def rmsnorm_reference(x, w, eps=1e-5, residual=None):
    """y = (x + residual) / sqrt(mean((x+residual)^2) + eps) * w ; returns (y, x + residual).
    Formula of the reference's RMSNorm module (interface_bindings/nn.py:224-238)."""
    h = x if residual is None else (x.float() + residual.float()).to(x.dtype)
    hf = h.float()
    y = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return y.to(x.dtype), h


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, residual, eps):
        d = x.shape[-1]
        x2 = x.reshape(-1, d).contiguous()
        T = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
        if residual is not None:
            r2 = residual.reshape(-1, d).contiguous()
            h = torch.empty_like(x2)
        else:
            r2, h = None, x2
        _lib.call("sx_rmsnorm_fwd", ptr(x2), ptr(r2), ptr(w), ptr(y), ptr(h if residual is not None else None),
                  ptr(rstd), c_ll(T), c_int(d), c_float(eps), stream())
        ctx.save_for_backward(h, w, rstd)
        ctx.has_res = residual is not None
        ctx.shape = x.shape
        return y.view(x.shape), (h.view(x.shape) if residual is not None else None)

    @staticmethod
    def backward(ctx, dy, dh):
        h, w, rstd = ctx.saved_tensors
        d = h.shape[-1]
        T = h.shape[0]
        dy2 = dy.reshape(-1, d).contiguous()
        dres = dh.reshape(-1, d).contiguous() if dh is not None else None
        dx = torch.empty_like(h)
        parts = _lib.lib().sx_rmsnorm_bwd_parts()
        scratch = torch.empty(parts * d, dtype=torch.float32, device=h.device)
        mg = getattr(w, "main_grad", None)
        if mg is not None:
            acc = getattr(w, "_main_grad_written", False)
            _lib.call("sx_rmsnorm_bwd", ptr(dy2), ptr(h), ptr(w), ptr(rstd), ptr(dres), ptr(dx), ptr(scratch),
                      ptr(mg if mg.dtype == torch.bfloat16 else None), ptr(mg if mg.dtype == torch.float32 else None),
                      c_int(int(acc)), c_ll(T), c_int(d), stream())
            w._main_grad_written = True
            dw = None
        else:
            dw = torch.empty_like(w)
            _lib.call("sx_rmsnorm_bwd", ptr(dy2), ptr(h), ptr(w), ptr(rstd), ptr(dres), ptr(dx), ptr(scratch),
                      ptr(dw), ptr(None), c_int(0), c_ll(T), c_int(d), stream())
        dx = dx.view(ctx.shape)
        return dx, dw, (dx if ctx.has_res else None), None


def rmsnorm(x, w, eps=1e-5, residual=None):
    """Returns (y, h) with h = x + residual (h is x itself when residual is None)."""
    if _native(x) and x.shape[-1] % 8 == 0:
        y, h = _RMSNormFn.apply(x, w, residual, eps)
        return y, (x if h is None else h)
    return rmsnorm_reference(x, w, eps, residual)


def layernorm(x, w, b=None, eps=1e-5):
    if _native(x) and not (torch.is_grad_enabled() and x.requires_grad):
        d = x.shape[-1]
        x2 = x.reshape(-1, d).contiguous()
        y = torch.empty_like(x2)
        _lib.call("sx_layernorm_fwd", ptr(x2), ptr(w), ptr(b), ptr(y), ptr(None), ptr(None), c_ll(x2.shape[0]),
                  c_int(d), c_float(eps), stream())
        return y.view(x.shape)
    if _native(x):
        from .aux import layernorm_train
        return layernorm_train(x, w, b, eps)
    return F.layer_norm(x, (x.shape[-1],), w, b, eps)


# ----------------------------------------------------------------------------- RoPE (R1)
def rope_tables(max_pos, dim, theta=10000.0, device=None, scaling=None, scale_factor=1.0):
    """cos/sin tables [max_pos, dim/2] (fp32). ``scaling``: None | 'linear' | 'ntk' | 'yarn' following the
    reference's context-extension rules (interface_bindings/model_zoo.py:998-1033)."""
    if scaling == "ntk":
        theta = theta * scale_factor
    elif scaling == "yarn":
        theta = theta * (scale_factor ** 0.8)
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim))
    pos = torch.arange(max_pos, dtype=torch.float32, device=device)
    if scaling == "linear":
        pos = pos / scale_factor
    ang = torch.outer(pos, inv)
    return ang.cos().contiguous(), ang.sin().contiguous()


def rope_reference(x, cos, sin, positions=None, interleaved=False):
    """x: [B, S, H, D]; rotate-half convention of the reference's Llama code
    (interface_bindings/llama_models.py:65-86); ``interleaved`` rotates adjacent pairs."""
    B, S, H, D = x.shape
    if positions is None:
        c, s = cos[:S], sin[:S]
        c = c.view(1, S, 1, D // 2)
        s = s.view(1, S, 1, D // 2)
    else:
        c = cos[positions].view(B, S, 1, D // 2)
        s = sin[positions].view(B, S, 1, D // 2)
    xf = x.float()
    if interleaved:
        x1, x2 = xf[..., 0::2], xf[..., 1::2]
        o = torch.stack((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1).flatten(-2)
    else:
        x1, x2 = xf[..., : D // 2], xf[..., D // 2:]
        o = torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1)
    return o.to(x.dtype)


class _RopeFn(torch.autograd.Function):
    """Rotation of the first ``heads`` heads of a [B, S, row] buffer (e.g. Q and K inside fused QKV). The kernel
    rotates in place; the autograd function hands it a private copy so no input is ever mutated."""

    @staticmethod
    def forward(ctx, x, cos, sin, positions, heads, D, interleaved):
        y = x.clone(memory_format=torch.contiguous_format)
        B, S = y.shape[0], y.shape[1]
        pos = positions.to(torch.int32).contiguous() if positions is not None else None
        _lib.call("sx_rope", ptr(y), ptr(cos), ptr(sin), ptr(pos), c_ll(B * S), c_int(S), c_int(heads), c_int(D),
                  c_ll(y.stride(1)), c_int(int(interleaved)), c_int(0), stream())
        ctx.save_for_backward(cos, sin, pos if pos is not None else torch.empty(0))
        ctx.meta = (heads, D, interleaved, pos is not None)
        return y

    @staticmethod
    def backward(ctx, dy):
        cos, sin, pos = ctx.saved_tensors
        heads, D, interleaved, has_pos = ctx.meta
        dx = dy.clone(memory_format=torch.contiguous_format)
        B, S = dx.shape[0], dx.shape[1]
        _lib.call("sx_rope", ptr(dx), ptr(cos), ptr(sin), ptr(pos if has_pos else None), c_ll(B * S), c_int(S),
                  c_int(heads), c_int(D), c_ll(dx.stride(1)), c_int(int(interleaved)), c_int(1), stream())
        return dx, None, None, None, None, None, None


def rope_qk_(qkv, cos, sin, n_rot_heads, head_dim, positions=None, interleaved=False):
    """Rotate the first ``n_rot_heads`` heads of a fused [B, S, (Hq+2Hk)*D] activation (Q then K heads)."""
    if _native(qkv):
        return _RopeFn.apply(qkv, cos, sin, positions, n_rot_heads, head_dim, interleaved)
    B, S, _ = qkv.shape
    rot = qkv[..., : n_rot_heads * head_dim].reshape(B, S, n_rot_heads, head_dim)
    rot = rope_reference(rot, cos, sin, positions, interleaved).reshape(B, S, -1)
    return torch.cat((rot, qkv[..., n_rot_heads * head_dim:]), dim=-1)


# ----------------------------------------------------------------------------- gated activations
GLU_ACT = {"silu": 0, "swiglu": 0, "gelu": 1, "geglu": 1, "relu": 2, "reglu": 2}


def glu_reference(gu, act="silu"):
    g, u = gu.float().chunk(2, dim=-1)
    a = {0: F.silu(g), 1: F.gelu(g, approximate="tanh"), 2: F.relu(g)}[GLU_ACT[act]]
    return (a * u).to(gu.dtype)


class _GluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu, act):
        Fd = gu.shape[-1] // 2
        g2 = gu.reshape(-1, 2 * Fd)
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        h = torch.empty(g2.shape[0], Fd, dtype=gu.dtype, device=gu.device)
        _lib.call("sx_glu_fwd", ptr(g2), ptr(h), c_ll(g2.shape[0]), c_int(Fd), c_int(act), stream())
        ctx.save_for_backward(g2)
        ctx.act = act
        ctx.shape = gu.shape
        return h.view(*gu.shape[:-1], Fd)

    @staticmethod
    def backward(ctx, dh):
        (g2,) = ctx.saved_tensors
        Fd = g2.shape[-1] // 2
        dh2 = dh.reshape(-1, Fd).contiguous()
        dgu = torch.empty_like(g2)
        _lib.call("sx_glu_bwd", ptr(dh2), ptr(g2), ptr(dgu), c_ll(g2.shape[0]), c_int(Fd), c_int(ctx.act), stream())
        return dgu.view(ctx.shape), None


def glu(gu, act="silu"):
    """act(gate) * up with gu = [..., 2F] laid out (gate | up)."""
    if _native(gu) and (gu.shape[-1] // 2) % 8 == 0:
        return _GluFn.apply(gu, GLU_ACT[act])
    return glu_reference(gu, act)


# ----------------------------------------------------------------------------- attention (A1/A2)
def attention_reference(q, k, v, causal=True, window=0, scale=None, return_lse=False):
    """q [B,Sq,Hq,D], k [B,Skv,Hk,D], v [B,Skv,Hv,D] -> [B,Sq,Hq,D]; fp32 softmax; GQA by head repetition.
    With Hv = Hk/2 two consecutive score heads share a V head (differential attention)."""
    B, Sq, Hq, D = q.shape
    Skv, Hk, Hv = k.shape[1], k.shape[2], v.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(Hq // Hk, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(Hq // Hv, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    off = Skv - Sq
    qi = torch.arange(Sq, device=q.device).view(-1, 1) + off
    ki = torch.arange(Skv, device=q.device).view(1, -1)
    mask = torch.zeros(Sq, Skv, dtype=torch.bool, device=q.device)
    if causal:
        mask |= ki > qi
    if window and window > 0:
        mask |= ki < qi - window + 1
    s = s.masked_fill(mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    p = torch.nan_to_num(p, nan=0.0)
    o = torch.matmul(p, vf).permute(0, 2, 1, 3).to(q.dtype)
    return (o, lse) if return_lse else o


def _attn_args(q, k, v, o, lse, causal, window, scale, v_head_div):
    a = _lib.SxAttnArgs()
    B, Sq, Hq, D = q.shape
    a.Q, a.K, a.V, a.O = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    a.lse = lse.data_ptr()
    a.q_row_stride, a.k_row_stride, a.v_row_stride, a.o_row_stride = q.stride(1), k.stride(1), v.stride(1), o.stride(1)
    a.q_batch_stride, a.k_batch_stride, a.v_batch_stride = q.stride(0), k.stride(0), v.stride(0)
    a.B, a.Sq, a.Skv, a.Hq, a.Hk, a.D = B, Sq, k.shape[1], Hq, k.shape[2], D
    a.v_head_div = v_head_div
    a.causal, a.window, a.scale = int(causal), int(window or 0), float(scale)
    a.status = _lib.status_word(q.device).data_ptr()
    return a


def _head_view_ok(t, D):
    return t.stride(3) == 1 and t.stride(2) == D and t.stride(1) % 8 == 0 and t.data_ptr() % 16 == 0


class _AttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, window, scale):
        B, Sq, Hq, D = q.shape
        q, k, v = [t if _head_view_ok(t, D) else t.contiguous() for t in (q, k, v)]
        v_head_div = k.shape[2] // v.shape[2]
        o = torch.empty(B, Sq, Hq, D, dtype=q.dtype, device=q.device)
        lse = torch.empty(B, Hq, Sq, dtype=torch.float32, device=q.device)
        a = _attn_args(q, k, v, o, lse, causal, window, scale, v_head_div)
        _lib.call("sx_attn_fwd", C.byref(a), stream())
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.meta = (causal, window, scale, v_head_div)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        causal, window, scale, v_head_div = ctx.meta
        dq, dk, dv = attention_backward(q, k, v, o, lse, do, causal, window, scale)
        return dq, dk, dv, None, None, None


def attention_backward_reference(q, k, v, o, lse, do, causal=True, window=0, scale=None):
    """fp32 gradients of attention given the forward's output and log-sum-exp. ``o`` and ``lse`` may be those of a
    softmax over MORE keys than ``k`` holds (ring / split-KV attention): the result is then this key block's share
    of dQ and its own dK, dV."""
    B, Sq, Hq, D = q.shape
    Skv, Hk, Hv = k.shape[1], k.shape[2], v.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(Hq // Hk, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(Hq // Hv, dim=1)
    dof = do.float().permute(0, 2, 1, 3)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    off = Skv - Sq
    qi = torch.arange(Sq, device=q.device).view(-1, 1) + off
    ki = torch.arange(Skv, device=q.device).view(1, -1)
    mask = torch.zeros(Sq, Skv, dtype=torch.bool, device=q.device)
    if causal:
        mask |= ki > qi
    if window and window > 0:
        mask |= ki < qi - window + 1
    p = torch.exp(s - lse.float().unsqueeze(-1)).masked_fill(mask, 0.0)
    p = torch.nan_to_num(p, nan=0.0, posinf=0.0)
    delta = (dof * o.float().permute(0, 2, 1, 3)).sum(-1, keepdim=True)
    dv = torch.matmul(p.transpose(-1, -2), dof)
    ds = p * (torch.matmul(dof, vf.transpose(-1, -2)) - delta)
    dq = torch.matmul(ds, kf) * scale
    dk = torch.matmul(ds.transpose(-1, -2), qf) * scale
    dk = dk.view(B, Hk, Hq // Hk, Skv, D).sum(2)
    dv = dv.view(B, Hv, Hq // Hv, Skv, D).sum(2)
    return (dq.permute(0, 2, 1, 3).to(q.dtype), dk.permute(0, 2, 1, 3).to(k.dtype), dv.permute(0, 2, 1, 3).to(v.dtype))


def attention_backward(q, k, v, o, lse, do, causal=True, window=0, scale=None):
    """(dQ, dK, dV) of flash attention from its saved output and log-sum-exp (natural log, [B, Hq, Sq]). Also the
    per-block step of ring attention backward: with the final ``o`` / ``lse`` of a softmax over all key blocks it
    returns this block's contribution."""
    B, Sq, Hq, D = q.shape
    Skv, Hk = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not (_native(q) and D == 128):
        return attention_backward_reference(q, k, v, o, lse, do, causal, window, scale)
    v_head_div = Hk // v.shape[2]
    q, k, v, o = [t if _head_view_ok(t, D) else t.contiguous() for t in (q, k, v, o)]
    lse = lse.contiguous()
    if v_head_div > 1:
        v_use = v.repeat_interleave(v_head_div, dim=2)
    else:
        v_use = v
    do = do if _head_view_ok(do, D) else do.contiguous()
    # dQ|dK|dV written into one fused buffer so that a fused QKV projection gets a contiguous grad
    dqkv = torch.empty(B, max(Sq, Skv), (Hq + 2 * Hk) * D, dtype=q.dtype, device=q.device) if Sq == Skv else None
    if dqkv is not None:
        dq = dqkv[..., : Hq * D].view(B, Sq, Hq, D)
        dk = dqkv[..., Hq * D: (Hq + Hk) * D].view(B, Skv, Hk, D)
        dv = dqkv[..., (Hq + Hk) * D:].view(B, Skv, Hk, D)
    else:
        dq = torch.empty(B, Sq, Hq, D, dtype=q.dtype, device=q.device)
        dk = torch.empty(B, Skv, Hk, D, dtype=q.dtype, device=q.device)
        dv = torch.empty(B, Skv, Hk, D, dtype=q.dtype, device=q.device)
    a = _attn_args(q, k, v_use, o, lse, causal, window, scale, 1)
    dq_acc = torch.empty(B, Hq, (Sq + 63) // 64 * 64, D, dtype=torch.float32, device=q.device)  # tiled by the kernel
    delta = torch.empty(B, Hq, Sq, dtype=torch.float32, device=q.device)
    a.dO, a.dQ, a.dK, a.dV = do.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.dq_accum, a.delta = dq_acc.data_ptr(), delta.data_ptr()
    a.do_row_stride = do.stride(1)
    a.dq_row_stride, a.dk_row_stride, a.dv_row_stride = dq.stride(1), dk.stride(1), dv.stride(1)
    a.dq_batch_stride, a.dk_batch_stride, a.dv_batch_stride = dq.stride(0), dk.stride(0), dv.stride(0)
    assert dq.stride(0) == Sq * dq.stride(1)
    _lib.call("sx_attn_bwd", C.byref(a), stream())
    if v_head_div > 1:
        dv = dv.view(B, Skv, Hk // v_head_div, v_head_div, D).sum(3)
    return dq, dk, dv


def attention(q, k, v, causal=True, window=0, scale=None):
    """Flash attention. q [B,Sq,Hq,D], k [B,Skv,Hk,D], v [B,Skv,Hv,D]; slices of a fused QKV tensor are
    consumed in place. head_dim 128 runs natively; head_dim 64 is zero-padded to 128 for training."""
    D = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if _native(q) and D in (64, 128):
        needs_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
        if D == 64 and needs_grad:
            pad = lambda t: F.pad(t, (0, 64))
            return _AttnFn.apply(pad(q), pad(k), pad(v), causal, window, scale)[..., :64]
        return _AttnFn.apply(q, k, v, causal, window, scale)
    return attention_reference(q, k, v, causal, window, scale)


def _expand_block_mask(block_mask, B, H, Sq, Skv, block=128):
    bm = block_mask.bool()
    while bm.dim() < 4:
        bm = bm.unsqueeze(0)
    bm = bm.expand(B if bm.shape[0] != 1 else 1, H if bm.shape[1] != 1 else 1, bm.shape[2], bm.shape[3])
    return bm.repeat_interleave(block, dim=2)[:, :, :Sq].repeat_interleave(block, dim=3)[..., :Skv]


def block_sparse_attention_reference(q, k, v, block_mask, causal=False, window=0, scale=None):
    """fp32 reference of ``block_sparse_attention``: tiles of 128 x 128 scores whose mask entry is False are removed."""
    B, Sq, Hq, D = q.shape
    Skv, Hk, Hv = k.shape[1], k.shape[2], v.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(Hq // Hk, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(Hq // Hv, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    off = Skv - Sq
    qi = torch.arange(Sq, device=q.device).view(-1, 1) + off
    ki = torch.arange(Skv, device=q.device).view(1, -1)
    drop = ~_expand_block_mask(block_mask.to(q.device), B, Hq, Sq, Skv)
    if causal:
        drop = drop | (ki > qi)
    if window and window > 0:
        drop = drop | (ki < qi - window + 1)
    s = s.masked_fill(drop, float("-inf"))
    p = torch.nan_to_num(torch.softmax(s, dim=-1), nan=0.0)
    return torch.matmul(p, vf).permute(0, 2, 1, 3).to(q.dtype)


@torch.no_grad()
def block_sparse_attention(q, k, v, block_mask, causal=False, window=0, scale=None):
    """Forward-only attention with a tile-level mask: ``block_mask`` [ceil(Sq/128), ceil(Skv/128)] (optionally with
    leading head and batch dimensions of size 1 or H / B), True where the 128 x 128 score tile takes part. Masked tiles
    are neither loaded nor multiplied by the kernel; causal / window masks still apply inside the tiles that remain.
    Query rows without any visible key give zeros. (Reference: kernel/algorithms/flex_attention.c:29-247 block masks,
    kernel/cuda/attention_cuda.cu:1154-1230 block-sparse kernel.)"""
    D = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    B, Sq, Hq, _ = q.shape
    Skv = k.shape[1]
    nq, nk = (Sq + 127) // 128, (Skv + 127) // 128
    assert block_mask.shape[-2:] == (nq, nk), f"block_mask must end in [{nq}, {nk}]"
    if not (_native(q) and D in (64, 128)):
        return block_sparse_attention_reference(q, k, v, block_mask, causal, window, scale)
    bm = block_mask.to(device=q.device)
    while bm.dim() < 4:
        bm = bm.unsqueeze(0)
    assert bm.shape[0] in (1, B) and bm.shape[1] in (1, Hq)
    bm = bm.to(torch.uint8).contiguous()
    q, k, v = [t if _head_view_ok(t, D) else t.contiguous() for t in (q, k, v)]
    o = torch.empty(B, Sq, Hq, D, dtype=q.dtype, device=q.device)
    lse = torch.empty(B, Hq, Sq, dtype=torch.float32, device=q.device)
    a = _attn_args(q, k, v, o, lse, causal, window, scale, k.shape[2] // v.shape[2])
    a.block_mask = bm.data_ptr()
    a.bm_batch_stride = bm.stride(0) if bm.shape[0] > 1 else 0
    a.bm_head_stride = bm.stride(1) if bm.shape[1] > 1 else 0
    _lib.call("sx_attn_fwd", C.byref(a), stream())
    return o


@torch.no_grad()
def attention_with_lse(q, k, v, causal=True, window=0, scale=None):
    """Forward only: (o [B,Sq,Hq,D], lse [B,Hq,Sq] natural log). The pair lets partial results over disjoint key
    sets be merged (ring / split-KV attention)."""
    D = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not (_native(q) and D == 128):
        return attention_reference(q, k, v, causal, window, scale, return_lse=True)
    B, Sq, Hq, _ = q.shape
    q, k, v = [t if _head_view_ok(t, D) else t.contiguous() for t in (q, k, v)]
    o = torch.empty(B, Sq, Hq, D, dtype=q.dtype, device=q.device)
    lse = torch.empty(B, Hq, Sq, dtype=torch.float32, device=q.device)
    a = _attn_args(q, k, v, o, lse, causal, window, scale, k.shape[2] // v.shape[2])
    _lib.call("sx_attn_fwd", C.byref(a), stream())
    return o, lse


def differential_attention(q, k, v, lam, causal=True, scale=None):
    """softmax(Q1 K1^T) V - lam * softmax(Q2 K2^T) V  (kernel/attention/differential_attention.c:25-27 states
    the intent). q, k: [B, S, 2H, D] with heads ordered (h0a, h0b, h1a, h1b, ..); v: [B, S, H, D]."""
    o = attention(q, k, v, causal=causal, scale=scale)  # two score heads share one V head
    B, S, H2, D = o.shape
    o = o.view(B, S, H2 // 2, 2, D)
    lam = lam if torch.is_tensor(lam) else torch.tensor(lam, device=o.device, dtype=o.dtype)
    return o[..., 0, :] - lam.to(o.dtype).view(1, 1, -1, 1) * o[..., 1, :]


# ----------------------------------------------------------------------------- cross entropy (L1)
def cross_entropy_reference(logits, target, ignore_index=-100):
    return F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), target.reshape(-1), ignore_index=ignore_index)


class _CEFn(torch.autograd.Function):
    """Mean CE over valid targets. The backward pass is computed in the forward kernel, in place in
    ``logits`` (which must not be used afterwards)."""

    @staticmethod
    def forward(ctx, logits, target, ignore_index):
        V = logits.shape[-1]
        l2 = logits.view(-1, V)
        T = l2.shape[0]
        tgt = target.reshape(-1).contiguous()
        loss = torch.empty(T, dtype=torch.float32, device=logits.device)
        inv = torch.empty(1, dtype=torch.float32, device=logits.device)
        _lib.call("sx_count_valid", ptr(tgt), c_ll(T), c_ll(ignore_index), ptr(inv), stream())
        grad = ctx.needs_input_grad[0]
        _lib.call("sx_cross_entropy", ptr(l2), c_int(int(l2.dtype == torch.float32)), ptr(tgt), ptr(loss), ptr(None),
                  c_ll(T), c_int(V), c_ll(l2.stride(0)), c_ll(ignore_index), ptr(inv), c_float(1.0), c_int(int(grad)),
                  stream())
        ctx.save_for_backward(logits)
        return loss.sum() * inv[0]

    @staticmethod
    def backward(ctx, g):
        (dlogits,) = ctx.saved_tensors
        return dlogits * g.to(dlogits.dtype), None, None


def cross_entropy(logits, target, ignore_index=-100):
    from . import debug as _dbg
    if _dbg.ENABLED:
        _dbg.check_indices(target, 0, logits.shape[-1], _dbg.SITE_CE_TARGET, also_ok=ignore_index)
    if logits.is_cuda and logits.dtype in (torch.bfloat16, torch.float32) and _lib.available() and \
            logits.is_contiguous():
        return _CEFn.apply(logits, target, ignore_index)
    return cross_entropy_reference(logits, target, ignore_index)


class _LinearCEFn(torch.autograd.Function):
    """Vocabulary projection + mean cross-entropy without ever holding [tokens, vocab] for the whole batch:
    tokens are processed in chunks; per chunk logits = h W^T (tcgen05 GEMM), the CE kernel turns them into
    gradients in place, and dh / dW GEMMs consume them immediately."""

    @staticmethod
    def forward(ctx, h, w, target, ignore_index, chunk):
        d = h.shape[-1]
        h2 = h.reshape(-1, d)
        T = h2.shape[0]
        V = w.shape[0]
        tgt = target.reshape(-1).contiguous()
        inv = torch.empty(1, dtype=torch.float32, device=h.device)
        _lib.call("sx_count_valid", ptr(tgt), c_ll(T), c_ll(ignore_index), ptr(inv), stream())
        loss = torch.empty(T, dtype=torch.float32, device=h.device)
        need_grad = ctx.needs_input_grad[0] or ctx.needs_input_grad[1]
        dh = torch.empty_like(h2) if need_grad else None
        mg = getattr(w, "main_grad", None)
        if need_grad:
            if mg is not None:
                dw, dw_init = mg, getattr(w, "_main_grad_written", False)
            else:
                dw, dw_init = torch.empty(V, d, dtype=torch.float32, device=h.device), False
        logits = torch.empty(min(chunk, T), V, dtype=torch.bfloat16, device=h.device)
        for t0 in range(0, T, chunk):
            t1 = min(t0 + chunk, T)
            lg = logits[: t1 - t0]
            gemm(h2[t0:t1], w, out=lg)
            _lib.call("sx_cross_entropy", ptr(lg), c_int(0), ptr(tgt[t0:t1]), ptr(loss[t0:t1]), ptr(None),
                      c_ll(t1 - t0), c_int(V), c_ll(lg.stride(0)), c_ll(ignore_index), ptr(inv), c_float(1.0),
                      c_int(int(need_grad)), stream())
            if need_grad:
                gemm(lg, w, b_mn=True, out=dh[t0:t1])
                gemm(lg, h2[t0:t1], a_mn=True, b_mn=True, out=dw, c=dw if dw_init else None,
                     beta=1.0 if dw_init else 0.0)
                dw_init = True
        if need_grad:
            if mg is not None:
                w._main_grad_written = True
                ctx.dw = None
            else:
                ctx.dw = dw
            ctx.save_for_backward(dh)
        ctx.hshape = h.shape
        ctx.wdtype = w.dtype
        return loss.sum() * inv[0]

    @staticmethod
    def backward(ctx, g):
        (dh,) = ctx.saved_tensors
        # g is 1 for a plain .backward() on the loss; other scalings are honoured by the multiply
        dhg = dh.view(ctx.hshape) * g.to(dh.dtype)
        dw = None if ctx.dw is None else (ctx.dw * g).to(ctx.wdtype)
        return dhg, dw, None, None, None


def linear_cross_entropy(h, w, target, ignore_index=-100, chunk=2048):
    """Mean next-token CE of logits = h @ w^T, vocab-chunk fused on GPU."""
    from . import debug as _dbg
    if _dbg.ENABLED:
        _dbg.check_indices(target, 0, w.shape[0], _dbg.SITE_CE_TARGET, also_ok=ignore_index)
    if _native(h) and w.shape[0] % 64 == 0 and h.shape[-1] % 64 == 0:
        return _LinearCEFn.apply(h, w, target, ignore_index, chunk)
    logits = F.linear(h, w)
    return cross_entropy_reference(logits, target, ignore_index)

"""Attention variants of the reference (kernel/attention/{attention,differential_attention,flex_attention}.c,
kernel/algorithms/{flash_attention,sparse_attention,swa}.c, kernel/position/{rope,yarn,alibi}.c; Python
``c_attention.py``: ``Attention``, ``DifferentialAttention``, ``FlexAttention``).

Causal / sliding-window / differential attention run on the tcgen05 flash kernels.  Variants whose scores carry an
arbitrary additive term or mask (ALiBi, block-sparse masks, score_mod callbacks, cross-attention over a different
key length) use a blockwise online-softmax formulation in PyTorch over key blocks, skipping fully masked blocks."""
from __future__ import annotations

import math

import torch
import torch.nn as tnn

from ..ops import functional as ops
from .modules import Linear, Module, RMSNorm


def alibi_slopes(num_heads: int, device=None):
    """Geometric head slopes 2^(-8 i / n) with the interpolation rule for non-power-of-two head counts
    (kernel/position/alibi.c)."""
    def pow2(n):
        start = 2.0 ** (-(2.0 ** -(math.log2(n) - 3)))
        return [start * start ** i for i in range(n)]
    if math.log2(num_heads).is_integer():
        s = pow2(num_heads)
    else:
        c = 2 ** math.floor(math.log2(num_heads))
        s = pow2(c) + pow2(2 * c)[0::2][: num_heads - c]
    return torch.tensor(s, dtype=torch.float32, device=device)


def alibi_bias(num_heads, q_len, k_len, device=None):
    """[H, q_len, k_len] bias  -slope * (i - j)  for j <= i (keys aligned to the end of the query range)."""
    i = torch.arange(q_len, device=device)[:, None] + (k_len - q_len)
    j = torch.arange(k_len, device=device)[None, :]
    return -alibi_slopes(num_heads, device)[:, None, None] * (i - j).clamp_min(0).float()


def yarn_tables(max_pos, dim, theta=10000.0, scale=4.0, original_max=4096, beta_fast=32.0, beta_slow=1.0, device=None):
    """YaRN cos/sin cache: per-frequency blend of interpolated and extrapolated RoPE with the 0.1 ln(s) + 1 attention
    temperature folded into the tables (kernel/position/yarn.c)."""
    return ops.rope_tables(max_pos, dim, theta, device, scaling="yarn", scale_factor=scale)


def blockwise_attention(q, k, v, *, bias=None, mask=None, score_mod=None, block_mask=None, block=128, scale=None,
                        causal=False):
    """Online-softmax attention over key blocks (the reference's 32x32 CPU flash loop, flash_attention.c:37-117, with
    device-sized blocks).  q [B, Sq, H, D], k/v [B, Sk, Hk, D].  ``bias`` broadcastable to [B, H, Sq, Sk]; ``mask``
    boolean keep-mask of that shape; ``score_mod(scores, b, h, q_idx, k_idx)``; ``block_mask`` boolean
    [ceil(Sq/block), ceil(Sk/block)] — blocks that are False are skipped without being computed."""
    B, Sq, H, D = q.shape
    Sk, Hk = k.shape[1], k.shape[2]
    scale = scale or 1.0 / math.sqrt(D)
    qf = q.permute(0, 2, 1, 3).float() * scale
    rep = H // Hk
    kf = k.permute(0, 2, 1, 3).float().repeat_interleave(rep, dim=1)
    vf = v.permute(0, 2, 1, 3).float().repeat_interleave(rep, dim=1)
    out = torch.zeros(B, H, Sq, v.shape[-1], device=q.device)
    m = torch.full((B, H, Sq, 1), -float("inf"), device=q.device)
    l = torch.zeros(B, H, Sq, 1, device=q.device)  # noqa: E741
    qi = torch.arange(Sq, device=q.device)[:, None] + (Sk - Sq if causal else 0)
    for kb, k0 in enumerate(range(0, Sk, block)):
        k1 = min(Sk, k0 + block)
        if block_mask is not None and not bool(block_mask[:, kb].any()):
            continue
        s = qf @ kf[:, :, k0:k1].transpose(-1, -2)
        kj = torch.arange(k0, k1, device=q.device)[None, :]
        if score_mod is not None:
            s = score_mod(s, None, None, qi, kj)
        if bias is not None:
            s = s + bias[..., k0:k1]
        keep = None
        if causal:
            keep = kj <= qi
        if mask is not None:
            mk = mask[..., k0:k1]
            keep = mk if keep is None else (keep & mk)
        if block_mask is not None:
            rows = block_mask[:, kb].repeat_interleave(block)[:Sq][:, None]
            keep = rows if keep is None else (keep & rows)
        if keep is not None:
            s = s.masked_fill(~keep, -float("inf"))
        m_new = torch.maximum(m, s.amax(-1, keepdim=True))
        m_safe = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)
        p = torch.exp(s - m_safe)
        alpha = torch.exp(torch.where(torch.isinf(m), torch.full_like(m, -float("inf")), m - m_safe))
        l = alpha * l + p.sum(-1, keepdim=True)  # noqa: E741
        out = alpha * out + p @ vf[:, :, k0:k1]
        m = m_new
    out = out / l.clamp_min(1e-30)
    return out.permute(0, 2, 1, 3).to(q.dtype)


class Attention(Module):
    """MHA / GQA with RoPE and an optional KV cache (attention.c:359-560)."""

    def __init__(self, d_model, num_heads, num_kv_heads=None, causal=True, window=0, rope_base=10000.0, bias=False,
                 dtype=None, device=None):
        super().__init__()
        self.H, self.Hk = num_heads, num_kv_heads or num_heads
        self.D = d_model // num_heads
        self.causal, self.window, self.rope_base = causal, window, rope_base
        self.qkv = Linear(d_model, (self.H + 2 * self.Hk) * self.D, bias=bias, dtype=dtype, device=device, init_std=0.02)
        self.out = Linear(d_model, d_model, bias=bias, dtype=dtype, device=device, init_std=0.02)
        self._rope = None

    def _tables(self, need, device):
        if self._rope is None or self._rope[0].shape[0] < need or self._rope[0].device != device:
            self._rope = ops.rope_tables(max(need, 256), self.D, self.rope_base, device)
        return self._rope

    def forward(self, x, kv_cache=None, start_pos=0):
        B, S, _ = x.shape
        H, Hk, D = self.H, self.Hk, self.D
        cos, sin = self._tables(start_pos + S, x.device)
        pos = torch.arange(start_pos, start_pos + S, device=x.device, dtype=torch.int32)
        qkv = ops.rope_qk_(self.qkv(x), cos, sin, H + Hk, D, pos if start_pos else None)
        q = qkv[..., : H * D].view(B, S, H, D)
        k = qkv[..., H * D:(H + Hk) * D].view(B, S, Hk, D)
        v = qkv[..., (H + Hk) * D:].view(B, S, Hk, D)
        if kv_cache is not None:
            if kv_cache.get("k") is not None:
                k = torch.cat([kv_cache["k"], k], 1)
                v = torch.cat([kv_cache["v"], v], 1)
            kv_cache["k"], kv_cache["v"] = k, v
        if k.shape[1] == S:
            o = ops.attention(q, k, v, causal=self.causal, window=self.window)
        else:
            o = blockwise_attention(q, k, v, causal=self.causal)
        return self.out(o.reshape(B, S, H * D))


class SlidingWindowAttention(Attention):
    """Causal attention restricted to the last ``window`` keys (kernel/algorithms/swa.c); the window bound is applied
    inside the flash kernel, so masked key tiles are never loaded."""

    def __init__(self, d_model, num_heads, window=4096, **kw):
        super().__init__(d_model, num_heads, causal=True, window=window, **kw)


class DifferentialAttention(Module):
    """softmax(Q1 K1^T) V - lambda softmax(Q2 K2^T) V with learnable lambda re-parameterisation and a per-head
    RMSNorm (differential_attention.c:25-27 states this intent; its body ignores lambda)."""

    def __init__(self, d_model, num_heads, lambda_init=0.8, causal=True, dtype=None, device=None):
        super().__init__()
        self.H, self.D = num_heads, d_model // num_heads // 2
        self.causal, self.lambda_init = causal, lambda_init
        self.qkv = Linear(d_model, 3 * d_model, bias=False, dtype=dtype, device=device, init_std=0.02)
        self.out = Linear(d_model, d_model, bias=False, dtype=dtype, device=device, init_std=0.02)
        mk = lambda: tnn.Parameter(torch.randn(self.D, device=device) * 0.1)  # noqa: E731
        self.lq1, self.lk1, self.lq2, self.lk2 = mk(), mk(), mk(), mk()
        self.norm = RMSNorm(2 * self.D, 1e-5, dtype=dtype, device=device)

    def lam(self):
        return torch.exp((self.lq1 * self.lk1).sum()) - torch.exp((self.lq2 * self.lk2).sum()) + self.lambda_init

    def forward(self, x):
        B, S, dm = x.shape
        H, D = self.H, self.D
        q, k, v = self.qkv(x).split(dm, dim=-1)
        q = q.reshape(B, S, 2 * H, D)
        k = k.reshape(B, S, 2 * H, D)
        v = v.reshape(B, S, H, 2 * D)
        lam = self.lam()
        # The kernel pairs two score heads with one value head of the same width: run it per value half.
        o = torch.cat([ops.differential_attention(q, k, v[..., :D].contiguous(), lam, causal=self.causal),
                       ops.differential_attention(q, k, v[..., D:].contiguous(), lam, causal=self.causal)], dim=-1)
        o = self.norm(o) * (1 - self.lambda_init)
        return self.out(o.reshape(B, S, dm))


class FlexAttention(Module):
    """Block-sparse mask + score-modification callback (flex_attention.c:29-247)."""

    def __init__(self, d_model, num_heads, block_size=128, dtype=None, device=None):
        super().__init__()
        self.H, self.D, self.block = num_heads, d_model // num_heads, block_size
        self.qkv = Linear(d_model, 3 * d_model, bias=False, dtype=dtype, device=device, init_std=0.02)
        self.out = Linear(d_model, d_model, bias=False, dtype=dtype, device=device, init_std=0.02)

    @staticmethod
    def create_block_mask(mask_fn, q_len, k_len, block, device=None):
        """Evaluates ``mask_fn(q_idx, k_idx) -> bool`` per element and keeps blocks with any True."""
        qi = torch.arange(q_len, device=device)[:, None]
        kj = torch.arange(k_len, device=device)[None, :]
        full = mask_fn(qi, kj)
        nq, nk = -(-q_len // block), -(-k_len // block)
        pad = torch.zeros(nq * block, nk * block, dtype=torch.bool, device=device)
        pad[:q_len, :k_len] = full
        return pad.view(nq, block, nk, block).any(3).any(1), full

    def forward(self, x, score_mod=None, mask_fn=None, context=None):
        B, S, dm = x.shape
        src = x if context is None else context
        q = self.qkv(x)[..., :dm].reshape(B, S, self.H, self.D)
        kv = self.qkv(src)[..., dm:]
        k, v = [t.reshape(B, src.shape[1], self.H, self.D) for t in kv.split(dm, dim=-1)]
        bm, full = (None, None)
        if mask_fn is not None:
            bm, full = self.create_block_mask(mask_fn, S, src.shape[1], self.block, x.device)
        o = blockwise_attention(q, k, v, score_mod=score_mod, mask=full, block_mask=None if bm is None else bm,
                                block=self.block)
        return self.out(o.reshape(B, S, dm))


class SparseAttention(FlexAttention):
    """Local window + strided global columns (kernel/algorithms/sparse_attention.c)."""

    def __init__(self, d_model, num_heads, local=128, stride=128, **kw):
        super().__init__(d_model, num_heads, **kw)
        self.local, self.stride = local, stride

    def forward(self, x):
        loc, st = self.local, self.stride
        return super().forward(x, mask_fn=lambda q, k: (k <= q) & ((q - k < loc) | (k % st == 0)))


class ALiBiAttention(FlexAttention):
    def forward(self, x):
        B, S, dm = x.shape
        q, k, v = [t.reshape(B, S, self.H, self.D) for t in self.qkv(x).split(dm, dim=-1)]
        o = blockwise_attention(q, k, v, bias=alibi_bias(self.H, S, S, x.device)[None], causal=True, block=self.block)
        return self.out(o.reshape(B, S, dm))


class CrossAttention(Module):
    """Queries from one stream, keys / values from another (the reference's multimodal cross-attention,
    flex_attention.c:150-200)."""

    def __init__(self, d_model, num_heads, d_context=None, dtype=None, device=None):
        super().__init__()
        self.H, self.D = num_heads, d_model // num_heads
        self.q = Linear(d_model, d_model, bias=False, dtype=dtype, device=device, init_std=0.02)
        self.kv = Linear(d_context or d_model, 2 * d_model, bias=False, dtype=dtype, device=device, init_std=0.02)
        self.out = Linear(d_model, d_model, bias=False, dtype=dtype, device=device, init_std=0.02)

    def forward(self, x, context, bias=None, mask=None):
        B, S, dm = x.shape
        q = self.q(x).reshape(B, S, self.H, self.D)
        k, v = [t.reshape(B, context.shape[1], self.H, self.D) for t in self.kv(context).split(dm, dim=-1)]
        if bias is None and mask is None and S == context.shape[1]:
            o = ops.attention(q, k, v, causal=False)
        else:
            o = blockwise_attention(q, k, v, bias=bias, mask=mask)
        return self.out(o.reshape(B, S, dm))


class MultiHeadLatentAttention(Module):
    """MLA (DeepSeek-V2): queries and keys/values pass through low-rank latents; a decoupled RoPE part of width
    ``rope_dim`` is shared by all heads (reference Python model, llama_models.py:447-536).  The KV cache holds only the
    latent (kv_lora_rank + rope_dim per token)."""

    def __init__(self, d_model, num_heads, kv_lora_rank=512, q_lora_rank=0, nope_dim=128, rope_dim=64, v_dim=128,
                 rope_base=10000.0, dtype=None, device=None):
        super().__init__()
        self.H, self.nope, self.rd, self.vd, self.rank = num_heads, nope_dim, rope_dim, v_dim, kv_lora_rank
        mk = lambda i, o: Linear(i, o, bias=False, dtype=dtype, device=device, init_std=0.02)  # noqa: E731
        if q_lora_rank:
            self.q_a, self.q_norm = mk(d_model, q_lora_rank), RMSNorm(q_lora_rank, dtype=dtype, device=device)
            self.q_b = mk(q_lora_rank, num_heads * (nope_dim + rope_dim))
        else:
            self.q_a, self.q_norm, self.q_b = None, None, mk(d_model, num_heads * (nope_dim + rope_dim))
        self.kv_a = mk(d_model, kv_lora_rank + rope_dim)
        self.kv_norm = RMSNorm(kv_lora_rank, dtype=dtype, device=device)
        self.kv_b = mk(kv_lora_rank, num_heads * (nope_dim + v_dim))
        self.out = mk(num_heads * v_dim, d_model)
        self.rope_base = rope_base
        self._rope = None

    def forward(self, x, latent_cache=None):
        B, S, _ = x.shape
        H, nd, rd, vd = self.H, self.nope, self.rd, self.vd
        q = self.q_b(x if self.q_a is None else self.q_norm(self.q_a(x))).view(B, S, H, nd + rd)
        lat = self.kv_a(x)                                            # [B, S, rank + rd]
        start = 0
        if latent_cache is not None:
            if latent_cache.get("latent") is not None:
                start = latent_cache["latent"].shape[1]
                lat_all = torch.cat([latent_cache["latent"], lat], 1)
            else:
                lat_all = lat
            latent_cache["latent"] = lat_all
        else:
            lat_all = lat
        Sk = lat_all.shape[1]
        if self._rope is None or self._rope[0].shape[0] < Sk or self._rope[0].device != x.device:
            self._rope = ops.rope_tables(max(Sk, 256), rd, self.rope_base, x.device)
        cos, sin = self._rope
        kv = self.kv_b(self.kv_norm(lat_all[..., : self.rank])).view(B, Sk, H, nd + vd)
        k_rope = ops.rope_reference(lat_all[..., self.rank:].view(B, Sk, 1, rd), cos, sin)
        q_rope = ops.rope_reference(q[..., nd:], cos, sin, torch.arange(start, start + S, device=x.device).expand(B, S))
        qf = torch.cat([q[..., :nd], q_rope.to(q.dtype)], -1)
        kf = torch.cat([kv[..., :nd], k_rope.to(kv.dtype).expand(B, Sk, H, rd)], -1)
        v = kv[..., nd:]
        scale = 1.0 / math.sqrt(nd + rd)
        if Sk == S and nd + rd == vd and vd in (64, 128):
            o = ops.attention(qf, kf, v, causal=True, scale=scale)
        else:
            o = blockwise_attention(qf, kf, v, causal=True, scale=scale)
        return self.out(o.reshape(B, S, H * vd))


class MixtureOfDepths(Module):
    """Routes the top ``capacity`` fraction of tokens through ``block`` and lets the rest skip it
    (the reference's mixture-of-depth router, flex_attention.c:202-247)."""

    def __init__(self, d_model, block: tnn.Module, capacity=0.5, dtype=None, device=None):
        super().__init__()
        self.router = Linear(d_model, 1, bias=False, dtype=dtype, device=device, init_std=0.02)
        self.block, self.capacity = block, capacity

    def forward(self, x):
        B, S, d = x.shape
        k = max(1, int(self.capacity * S))
        score = self.router(x).squeeze(-1).float()
        top = torch.topk(score, k, dim=-1).indices.sort(-1).values              # keep sequence order
        sel = torch.gather(x, 1, top[..., None].expand(B, k, d))
        upd = self.block(sel) * torch.sigmoid(torch.gather(score, 1, top))[..., None].to(x.dtype)
        return x.scatter_add(1, top[..., None].expand(B, k, d), upd)

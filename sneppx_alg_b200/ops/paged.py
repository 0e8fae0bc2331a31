"""A3/A4 front-ends: paged KV cache append (+RoPE) and paged decode attention, with PyTorch references."""
from __future__ import annotations

import math
import os

import torch

from . import _lib
from ._lib import c_float, c_int, c_ll, ptr, stream
from .functional import rope_reference


def kv_append_reference(qkv, cos, sin, pos, slot, k_cache, v_cache, Hq, Hkv, D, rotate=True):
    T = qkv.shape[0]
    x = qkv.view(T, Hq + 2 * Hkv, D)
    if rotate:
        rot = rope_reference(x[:, : Hq + Hkv].unsqueeze(0), cos, sin, pos.view(1, T).long())[0]
        x[:, : Hq + Hkv] = rot
    ok = slot >= 0
    kc = k_cache.view(-1, Hkv, D)
    vc = v_cache.view(-1, Hkv, D)
    kc[slot[ok].long()] = x[ok, Hq: Hq + Hkv]
    vc[slot[ok].long()] = x[ok, Hq + Hkv:]
    return qkv


def kv_append_(qkv, cos, sin, pos, slot, k_cache, v_cache, Hq, Hkv, D, rotate=True):
    """In place: rotate Q and K rows of ``qkv`` [T, (Hq+2Hkv)*D] and scatter K/V into the block pool at ``slot``."""
    if qkv.is_cuda and qkv.dtype == torch.bfloat16 and _lib.available():
        from . import debug as _dbg
        if _dbg.ENABLED:
            _dbg.check_indices(slot, -1, k_cache.shape[0] * k_cache.shape[1], _dbg.SITE_KV_SLOT)
        _lib.call("sx_kv_append", ptr(qkv), c_ll(qkv.stride(0)), ptr(cos), ptr(sin), ptr(pos.to(torch.int32)),
                  ptr(slot.to(torch.int32)), ptr(k_cache), ptr(v_cache), c_int(qkv.shape[0]), c_int(Hq), c_int(Hkv),
                  c_int(D), c_int(int(rotate)), stream())
        return qkv
    return kv_append_reference(qkv, cos, sin, pos, slot, k_cache, v_cache, Hq, Hkv, D, rotate)


def paged_decode_reference(q, k_cache, v_cache, block_table, seq_lens, scale=None):
    """q [B, Hq, D]; caches [blocks, bs, Hkv, D]; block_table [B, max_blocks]; seq_lens [B]."""
    B, Hq, D = q.shape
    bs, Hkv = k_cache.shape[1], k_cache.shape[2]
    scale = scale or 1.0 / math.sqrt(D)
    out = torch.zeros(B, Hq, D, dtype=torch.float32, device=q.device)
    for b in range(B):
        n = int(seq_lens[b])
        if n == 0:
            continue
        blocks = block_table[b, : (n + bs - 1) // bs].long()
        k = k_cache[blocks].reshape(-1, Hkv, D)[:n].float().repeat_interleave(Hq // Hkv, dim=1)
        v = v_cache[blocks].reshape(-1, Hkv, D)[:n].float().repeat_interleave(Hq // Hkv, dim=1)
        s = torch.einsum("hd,nhd->hn", q[b].float(), k) * scale
        out[b] = torch.einsum("hn,nhd->hd", torch.softmax(s, -1), v)
    return out.to(q.dtype)


def _use_tc(D, bs, G) -> bool:
    """Tensor-core decode kernel: head size 128, block size a divisor of 128 (>= 8), at most 8 query heads per KV
    head. ``SX_PAGED_TC=0`` selects the SIMT kernel."""
    return D == 128 and bs >= 8 and 128 % bs == 0 and G <= 8 and os.environ.get("SX_PAGED_TC", "1") != "0"


def paged_decode(q, k_cache, v_cache, block_table, seq_lens, scale=None):
    B, Hq, D = q.shape
    bs, Hkv = k_cache.shape[1], k_cache.shape[2]
    scale = scale or 1.0 / math.sqrt(D)
    if q.is_cuda and q.dtype == torch.bfloat16 and _lib.available() and D in (64, 128) and Hq // Hkv <= 8:
        q = q if q.stride(2) == 1 and q.stride(1) == D else q.contiguous()
        from . import debug as _dbg
        if _dbg.ENABLED:
            _dbg.check_indices(block_table, 0, k_cache.shape[0], _dbg.SITE_BLOCK_TABLE)
        max_len = block_table.shape[1] * bs
        tc = _use_tc(D, bs, Hq // Hkv) and k_cache.is_contiguous() and v_cache.is_contiguous()
        if tc:
            ns = _lib.lib().sx_paged_decode_tc_splits(c_int(max_len), c_int(B * Hkv))
        else:
            ns = _lib.lib().sx_paged_decode_splits2(c_int(max_len), c_int(B * Hkv))
        out = torch.empty(B, Hq, D, dtype=q.dtype, device=q.device)
        if _dbg.ENABLED:
            _dbg.poison_(out)
        o_part = torch.empty(B * Hq * ns * D, dtype=torch.float32, device=q.device)
        ml = torch.empty(B * Hq * ns * 2, dtype=torch.float32, device=q.device)
        if tc:
            _lib.call("sx_paged_decode_tc", ptr(q), c_ll(q.stride(0)), ptr(k_cache), ptr(v_cache),
                      c_ll(k_cache.shape[0]), ptr(block_table.to(torch.int32).contiguous()),
                      ptr(seq_lens.to(torch.int32).contiguous()), ptr(out), c_ll(out.stride(0)), ptr(o_part), ptr(ml),
                      c_int(B), c_int(Hq), c_int(Hkv), c_int(D), c_int(bs), c_int(block_table.shape[1]), c_int(ns),
                      c_float(scale), ptr(_lib.status_word(q.device)), stream())
            return out
        _lib.call("sx_paged_decode", ptr(q), c_ll(q.stride(0)), ptr(k_cache), ptr(v_cache),
                  ptr(block_table.to(torch.int32).contiguous()), ptr(seq_lens.to(torch.int32).contiguous()), ptr(out),
                  c_ll(out.stride(0)), ptr(o_part), ptr(ml), c_int(B), c_int(Hq), c_int(Hkv), c_int(D), c_int(bs),
                  c_int(block_table.shape[1]), c_int(ns), c_float(scale), stream())
        return out
    return paged_decode_reference(q, k_cache, v_cache, block_table, seq_lens, scale)

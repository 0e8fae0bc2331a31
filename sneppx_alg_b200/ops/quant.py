"""Q1 front-ends: block-scaled fp8 (e4m3) and INT4 group quantisation with their dequantisers; PyTorch
restatements serve CPU tensors and act as the oracle. Formats: activations 1x128 scales, weights 128x128 scales
(fp32), INT4 symmetric with group 128 along K packed two per byte (low nibble first, offset 8).
Reference API names: ``quantize_fp8_e4m3`` / ``quantize_int4`` (interface_bindings/quantization.py)."""
from __future__ import annotations

import torch

from . import _lib
from ._lib import c_int, c_ll, ptr, stream

E4M3_MAX = 448.0


def _native(x):
    return x.is_cuda and x.dtype == torch.bfloat16 and _lib.available()


def quant_fp8_1x128_reference(x):
    T, K = x.shape
    xb = x.float().view(T, K // 128, 128)
    amax = xb.abs().amax(-1)
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (xb / scale[..., None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(T, K)
    return q, scale


def quant_fp8_1x128(x):
    """x bf16 [T, K] (K % 128 == 0) -> (q float8_e4m3fn [T, K], scales fp32 [T, K/128])."""
    if _native(x) and x.shape[1] % 128 == 0:
        x = x.contiguous()
        T, K = x.shape
        q = torch.empty(T, K, dtype=torch.uint8, device=x.device)
        s = torch.empty(T, K // 128, dtype=torch.float32, device=x.device)
        _lib.call("sx_quant_fp8_1x128", ptr(x), ptr(q), ptr(s), c_ll(T), c_int(K), stream())
        return q.view(torch.float8_e4m3fn), s
    return quant_fp8_1x128_reference(x)


def quant_fp8_128x128_reference(w):
    N, K = w.shape
    nb, kb = (N + 127) // 128, (K + 127) // 128
    wp = torch.zeros(nb * 128, kb * 128, dtype=torch.float32, device=w.device)
    wp[:N, :K] = w.float()
    blk = wp.view(nb, 128, kb, 128).permute(0, 2, 1, 3)
    amax = blk.abs().amax((-1, -2))
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (blk / scale[..., None, None]).clamp(-E4M3_MAX, E4M3_MAX).permute(0, 2, 1, 3).reshape(nb * 128, kb * 128)
    return q[:N, :K].contiguous().to(torch.float8_e4m3fn), scale


def quant_fp8_128x128(w):
    """w bf16 [N, K] -> (q float8_e4m3fn [N, K], scales fp32 [ceil(N/128), ceil(K/128)])."""
    if _native(w):
        w = w.contiguous()
        N, K = w.shape
        q = torch.empty(N, K, dtype=torch.uint8, device=w.device)
        s = torch.empty((N + 127) // 128, (K + 127) // 128, dtype=torch.float32, device=w.device)
        _lib.call("sx_quant_fp8_128x128", ptr(w), ptr(q), ptr(s), c_int(N), c_int(K), stream())
        return q.view(torch.float8_e4m3fn), s
    return quant_fp8_128x128_reference(w)


def dequant_fp8(q, scales, block="1x128", dtype=torch.bfloat16):
    rows, K = q.shape
    if q.is_cuda and _lib.available() and dtype == torch.bfloat16:
        out = torch.empty(rows, K, dtype=torch.bfloat16, device=q.device)
        _lib.call("sx_dequant_fp8", ptr(q.contiguous()), ptr(scales.contiguous()), ptr(out), c_ll(rows), c_int(K),
                  c_int(0 if block == "1x128" else 1), stream())
        return out
    qf = q.float()
    if block == "1x128":
        s = scales.repeat_interleave(128, dim=1)[:, :K]
    else:
        s = scales.repeat_interleave(128, dim=0)[:rows].repeat_interleave(128, dim=1)[:, :K]
    return (qf * s).to(dtype)


def quant_int4_reference(w):
    N, K = w.shape
    wb = w.float().view(N, K // 128, 128)
    amax = wb.abs().amax(-1)
    scale = torch.where(amax > 0, amax / 7.0, torch.ones_like(amax))
    q = torch.round(wb / scale[..., None]).clamp(-8, 7).to(torch.int32).view(N, K) + 8
    packed = (q[:, 0::2] | (q[:, 1::2] << 4)).to(torch.uint8)
    return packed, scale


def quant_int4(w):
    """w bf16 [N, K] (K % 128 == 0) -> (packed uint8 [N, K/2], scales fp32 [N, K/128])."""
    if _native(w) and w.shape[1] % 128 == 0:
        w = w.contiguous()
        N, K = w.shape
        p = torch.empty(N, K // 2, dtype=torch.uint8, device=w.device)
        s = torch.empty(N, K // 128, dtype=torch.float32, device=w.device)
        _lib.call("sx_quant_int4", ptr(w), ptr(p), ptr(s), c_ll(N), c_int(K), stream())
        return p, s
    return quant_int4_reference(w)


def dequant_int4(packed, scales, dtype=torch.bfloat16):
    N, K2 = packed.shape
    K = K2 * 2
    if packed.is_cuda and _lib.available() and dtype == torch.bfloat16:
        out = torch.empty(N, K, dtype=torch.bfloat16, device=packed.device)
        _lib.call("sx_dequant_int4", ptr(packed.contiguous()), ptr(scales.contiguous()), ptr(out), c_ll(N), c_int(K),
                  stream())
        return out
    lo = (packed & 15).to(torch.int32) - 8
    hi = (packed >> 4).to(torch.int32) - 8
    q = torch.stack([lo, hi], dim=-1).view(N, K).float()
    return (q * scales.repeat_interleave(128, dim=1)).to(dtype)

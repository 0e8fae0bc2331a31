"""Q1 front-ends: block-scaled fp8 (e4m3) and INT4 group quantisation with their dequantisers; PyTorch
restatements serve CPU tensors and act as the oracle. Formats: activations 1x128 scales, weights 128x128 scales
(fp32), INT4 symmetric with group 128 along K packed two per byte (low nibble first, offset 8).
Reference API names: ``quantize_fp8_e4m3`` / ``quantize_int4`` (interface_bindings/quantization.py)."""
from __future__ import annotations

import ctypes

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


# ----------------------------------------------------------------------------- Q2 dequant-GEMM
def gemm_fp8_reference(xq, sx, wq, sw, bias=None, out_dtype=torch.bfloat16):
    """fp32 oracle of the block-scaled product: dequantise both operands, multiply."""
    M, K = xq.shape
    N = wq.shape[0]
    x = xq.float().view(M, K // 128, 128) * sx.float()[..., None]
    w = dequant_fp8(wq, sw, "128x128", torch.float32)
    y = x.view(M, K) @ w.t()
    if bias is not None:
        y = y + bias.float()
    return y.to(out_dtype)


def gemm_fp8(x, wq, sw, bias=None, xq=None, sx=None):
    """y = x @ W^T with both operands in block-scaled e4m3 on the fp8 tensor-core path.

    x bf16 [.., K] is quantised per 1 x 128 block on the fly (or pass ``xq`` / ``sx``); ``wq`` float8_e4m3fn [N, K] with
    ``sw`` fp32 [ceil(N/128), K/128] (``quant_fp8_128x128``). Weights are streamed once; suited to decode-size M as
    well as expert GEMMs."""
    K = x.shape[-1] if x is not None else xq.shape[-1]
    lead = x.shape[:-1] if x is not None else xq.shape[:-1]
    if xq is None:
        xq, sx = quant_fp8_1x128(x.reshape(-1, K))
    M, N = xq.shape[0], wq.shape[0]
    if xq.is_cuda and _lib.available() and K % 128 == 0 and M <= 256:
        xq_, wq_ = xq.view(torch.uint8).contiguous(), wq.view(torch.uint8).contiguous()
        out = torch.empty(M, N, dtype=torch.bfloat16, device=xq.device)
        fn = _lib.lib().sx_gemm_fp8_workspace
        fn.restype = ctypes.c_longlong
        nbytes = fn(c_int(M), c_int(N), c_int(K))
        work = torch.empty(max(nbytes // 4, 1), dtype=torch.float32, device=xq.device) if nbytes else None
        b = bias.float().contiguous() if bias is not None else None
        _lib.call("sx_gemm_fp8", ptr(xq_), c_ll(xq_.stride(0)), ptr(sx.contiguous()), ptr(wq_), c_ll(wq_.stride(0)),
                  ptr(sw.contiguous()), ptr(b), ptr(out), c_ll(out.stride(0)), ptr(work), c_int(M), c_int(N), c_int(K),
                  ptr(_lib.status_word(xq.device)), stream())
        return out.view(*lead, N)
    if xq.is_cuda and _lib.available() and K % 128 == 0:
        # large M: the swap-AB kernel would re-read the weights per 128-token tile; expand the weights inside the bf16 GEMM
        xb = dequant_fp8(xq, sx, "1x128", torch.bfloat16)
        return gemm_dequant(xb, wq, sw, "fp8", bias).view(*lead, N)
    return gemm_fp8_reference(xq, sx, wq, sw, bias).view(*lead, N)


def gemm_fp8_grouped_reference(x, tile_group, W):
    """Oracle of ``gemm_fp8_grouped``: both operands rounded to block-scaled e4m3 (1 x 128 rows of ``x``, 128 x 128
    blocks of each expert's matrix), de-quantised to fp32, multiplied per 128-row tile with the tile's expert."""
    E, N, K = W.shape
    xq, sx = quant_fp8_1x128_reference(x.reshape(-1, K))
    wq, sw = quant_fp8_128x128_reference(W.reshape(E * N, K))
    xd = dequant_fp8(xq, sx, "1x128", torch.float32)
    wd = dequant_fp8(wq, sw, "128x128", torch.float32).view(E, N, K)
    out = torch.zeros(x.shape[0], N, dtype=torch.float32, device=x.device)
    tg = tile_group.tolist()
    for t, e in enumerate(tg[: x.shape[0] // 128]):
        if e >= 0:
            out[t * 128:(t + 1) * 128] = xd[t * 128:(t + 1) * 128] @ wd[e].t()
    return out.to(x.dtype)


def gemm_fp8_grouped(x, tile_group, W, wq=None, sw=None):
    """Expert-sorted rows ``x`` [rows, K] (bf16, segments padded to 128 rows) times the stacked expert matrices
    ``W`` [E, N, K], tile t using expert ``tile_group[t]`` (-1: output rows zero), with both operands in
    block-scaled e4m3 on the fp8 tensor-core path (G2 in fp8). ``wq`` / ``sw`` may carry the experts already
    quantised (``quant_fp8_128x128`` of ``W.view(E * N, K)``). N and K must be multiples of 128."""
    E, N, K = W.shape
    rows = x.shape[0]
    if not (x.is_cuda and x.dtype == torch.bfloat16 and _lib.available()):
        return gemm_fp8_grouped_reference(x, tile_group, W)
    if N % 128 or K % 128 or rows % 128:
        raise ValueError(f"gemm_fp8_grouped: rows {rows}, N {N}, K {K} must be multiples of 128")
    xq, sx = quant_fp8_1x128(x)
    if wq is None:
        wq, sw = quant_fp8_128x128(W.reshape(E * N, K))
    out = torch.empty(rows, N, dtype=torch.bfloat16, device=x.device)
    xq_, wq_ = xq.view(torch.uint8), wq.view(torch.uint8)
    _lib.call("sx_gemm_fp8_grouped", ptr(xq_), c_ll(xq_.stride(0)), ptr(sx.contiguous()), ptr(wq_), c_ll(wq_.stride(0)),
              ptr(sw.contiguous()), ptr(tile_group), c_int(E), ptr(out), c_ll(out.stride(0)), c_int(rows), c_int(N),
              c_int(K), ptr(_lib.status_word(x.device)), stream())
    return out


def gemm_dequant(x, qweight, scales, mode="fp8", bias=None):
    """y = x @ dequant(W)^T. x bf16 [.., K]; mode 'fp8': qweight float8_e4m3fn/uint8 [N, K], scales [N/128, K/128];
    mode 'int4': qweight uint8 [N, K/2], scales [N, K/128]. CUDA: weights are expanded to bf16 inside the GEMM."""
    K = x.shape[-1]
    x2 = x.reshape(-1, K)
    N = qweight.shape[0]
    if x.is_cuda and x.dtype == torch.bfloat16 and _lib.available() and K % 128 == 0:
        x2 = x2.contiguous()
        out = torch.empty(x2.shape[0], N, dtype=torch.bfloat16, device=x.device)
        b = bias.float().contiguous() if bias is not None else None
        _lib.call("sx_gemm_dequant", ptr(x2), c_ll(x2.stride(0)), ptr(qweight), ptr(scales.contiguous()), ptr(b),
                  ptr(out), c_ll(out.stride(0)), c_int(x2.shape[0]), c_int(N), c_int(K),
                  c_int(0 if mode == "fp8" else 1), ptr(_lib.status_word(x.device)), stream())
        return out.view(*x.shape[:-1], N)
    w = dequant_fp8(qweight.view(torch.float8_e4m3fn) if qweight.dtype == torch.uint8 else qweight, scales, "128x128",
                    torch.float32) if mode == "fp8" else dequant_int4(qweight, scales, torch.float32)
    y = x2.float() @ w.t()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype).view(*x.shape[:-1], N)


class QuantizedLinear(torch.nn.Module):
    """Weight-only quantised linear layer (fp8 e4m3 128x128-block scales, or INT4 group 128); the reference's
    ``QuantizedLinear`` (interface_bindings/quantization.py) dequantises in NumPy before a dense matmul."""

    def __init__(self, weight, mode="fp8", bias=None, fp8_activations=True):
        super().__init__()
        self.mode = mode
        # fp8 mode, up to 256 rows (decode and small prefill chunks): quantise the activations per 1 x 128 block and run
        # the fp8 x fp8 tensor-core GEMM, which streams the weights once; larger inputs expand the weights to bf16 inside
        # the GEMM (weight-only).
        self.fp8_activations = fp8_activations
        self.out_features, self.in_features = weight.shape
        w = weight.detach().to(torch.bfloat16)
        if mode == "fp8":
            q, s = quant_fp8_128x128(w)
            q = q.view(torch.uint8)
        else:
            q, s = quant_int4(w)
        self.register_buffer("qweight", q)
        self.register_buffer("scales", s)
        self.bias = None if bias is None else torch.nn.Parameter(bias.detach().clone(), requires_grad=False)

    @classmethod
    def from_linear(cls, lin, mode="fp8"):
        return cls(lin.weight, mode, getattr(lin, "bias", None))

    def forward(self, x):
        if self.mode == "fp8" and self.fp8_activations and x.is_cuda and x.dtype == torch.bfloat16 \
                and x.numel() // x.shape[-1] <= 256 and _lib.available():
            return gemm_fp8(x, self.qweight, self.scales, self.bias)
        rows = x.numel() // x.shape[-1]
        if rows > 256 and x.is_cuda and x.dtype == torch.bfloat16 and _lib.available():
            # prefill-size inputs: expanding the weight once (a bandwidth-bound pass over N x K) and running the bf16
            # tensor-core GEMM beats expanding it inside the GEMM, whose converter warps cap it far below the MMA rate
            from .gemm import gemm
            w = dequant_fp8(self.qweight, self.scales, "128x128") if self.mode == "fp8" else dequant_int4(self.qweight, self.scales)
            y = gemm(x.reshape(rows, x.shape[-1]), w)
            if self.bias is not None:
                y = y + self.bias.to(y.dtype)
            return y.view(*x.shape[:-1], self.out_features)
        return gemm_dequant(x, self.qweight, self.scales, self.mode, self.bias)


def quantize_model_(model, mode="fp8", min_features=128, skip=("lm_head", "router")):
    """Replace every large ``Linear`` by a ``QuantizedLinear`` in place (serving)."""
    from ..nn.modules import Linear
    for name, mod in list(model.named_modules()):
        for cname, child in list(mod.named_children()):
            if isinstance(child, (Linear, torch.nn.Linear)) and child.weight.shape[1] % 128 == 0 \
                    and min(child.weight.shape) >= min_features and not any(s in cname for s in skip):
                setattr(mod, cname, QuantizedLinear.from_linear(child, mode))
    return model

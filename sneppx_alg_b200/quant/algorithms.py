"""Quantisation algorithms (the reference's ``quantization.py``: ``QuantMode``, int8 / int4 / fp8, ``awq_quantize``,
``gptq_quantize``; C twins kernel/quantization/{quantize_int8,quantize_fp8,awq,gptq}.c; ``mx_formats.py``: MXFP8/6/4
with 32-element E8M0 block scales and NVFP4).  Everything is vectorised torch code that runs on the GPU when the
tensors live there; the serving-path kernels (fp8 1x128 / 128x128, int4 group-128 dequant-GEMM) are in ``ops.quant``."""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass

import torch


class QuantMode(enum.Enum):
    INT8_SYMMETRIC = "int8_sym"
    INT8_ASYMMETRIC = "int8_asym"
    INT8_PER_CHANNEL = "int8_channel"
    INT4 = "int4"
    FP8_E4M3 = "fp8_e4m3"
    FP8_E5M2 = "fp8_e5m2"


# ---- INT8 / INT4
def quantize_int8(w, mode=QuantMode.INT8_SYMMETRIC):
    """Returns (q int8 / uint8, scale, zero_point)."""
    wf = w.float()
    if mode == QuantMode.INT8_SYMMETRIC:
        scale = wf.abs().max().clamp_min(1e-12) / 127.0
        return torch.round(wf / scale).clamp(-127, 127).to(torch.int8), scale, torch.zeros((), device=w.device)
    if mode == QuantMode.INT8_PER_CHANNEL:
        scale = wf.abs().amax(dim=tuple(range(1, w.dim())), keepdim=True).clamp_min(1e-12) / 127.0
        return torch.round(wf / scale).clamp(-127, 127).to(torch.int8), scale, torch.zeros_like(scale)
    if mode == QuantMode.INT8_ASYMMETRIC:
        lo, hi = wf.min(), wf.max()
        scale = ((hi - lo) / 255.0).clamp_min(1e-12)
        zp = torch.round(-lo / scale).clamp(0, 255)
        return (torch.round(wf / scale) + zp).clamp(0, 255).to(torch.uint8), scale, zp
    raise ValueError(mode)


def dequantize_int8(q, scale, zero_point=0.0):
    return (q.float() - zero_point) * scale


def quantize_int4_packed(w, group=128):
    """Symmetric int4 in groups along the last dim; two nibbles per byte (low nibble first), values offset by 8."""
    wf = w.float()
    K = wf.shape[-1]
    assert K % group == 0 and K % 2 == 0
    g = wf.reshape(*wf.shape[:-1], K // group, group)
    scale = g.abs().amax(-1, keepdim=True).clamp_min(1e-12) / 7.0
    q = (torch.round(g / scale).clamp(-8, 7) + 8).to(torch.uint8).reshape(*wf.shape)
    return (q[..., 0::2] | (q[..., 1::2] << 4)), scale.squeeze(-1)


def dequantize_int4_packed(packed, scale, group=128):
    lo, hi = (packed & 0xF).float() - 8, (packed >> 4).float() - 8
    q = torch.stack([lo, hi], -1).flatten(-2)
    return (q.reshape(*q.shape[:-1], -1, group) * scale.unsqueeze(-1)).reshape(q.shape)


# ---- FP8 (bit-exact through torch's float8 dtypes: round-to-nearest-even, saturating)
_F8 = {QuantMode.FP8_E4M3: (torch.float8_e4m3fn, 448.0), QuantMode.FP8_E5M2: (torch.float8_e5m2, 57344.0)}


def fp8_encode(x, mode=QuantMode.FP8_E4M3):
    dt, mx = _F8[mode]
    return x.float().clamp(-mx, mx).to(dt).view(torch.uint8)


def fp8_decode(bits, mode=QuantMode.FP8_E4M3):
    return bits.view(_F8[mode][0]).float()


def quantize_fp8(w, mode=QuantMode.FP8_E4M3):
    mx = _F8[mode][1]
    scale = w.float().abs().max().clamp_min(1e-12) / mx
    return fp8_encode(w.float() / scale, mode), scale


# ---- AWQ: per-input-channel scales from activation magnitudes, grid search over the exponent
def awq_quantize(w, act_scale, n_grid=20, group=128, bits=4):
    """w [out, in], act_scale [in] (mean |activation|).  Searches s = act_scale^a, a in [0, 1), minimising the output
    error of quantising (w * s) and dividing the activation by s (awq.c).  Returns (w_q dequantised, s, best a)."""
    wf, a_s = w.float(), act_scale.float().clamp_min(1e-8)
    qmax = 2 ** (bits - 1) - 1

    def fake_q(m):
        g = m.reshape(m.shape[0], -1, group)
        sc = g.abs().amax(-1, keepdim=True).clamp_min(1e-12) / qmax
        return (torch.round(g / sc).clamp(-qmax - 1, qmax) * sc).reshape(m.shape)

    best = (float("inf"), None, None, 0.0)
    for i in range(n_grid):
        a = i / n_grid
        s = a_s.pow(a)
        s = s / (s.max() * s.min()).sqrt()
        wq = fake_q(wf * s) / s
        err = float((((wq - wf) * a_s) ** 2).mean())
        if err < best[0]:
            best = (err, wq, s, a)
    return best[1].to(w.dtype), best[2], best[3]


# ---- GPTQ: column-by-column quantisation with Hessian-weighted error propagation
def gptq_quantize(w, x, bits=4, group=128, damp=0.01, block=128):
    """w [out, in]; x [n, in] calibration inputs.  H = 2 X^T X + damp * mean(diag) I; columns are quantised in order
    and the error is pushed onto the not-yet-quantised columns through the Cholesky factor of H^-1 (gptq.c)."""
    W = w.float().clone()
    n_in = W.shape[1]
    H = 2.0 * x.float().T @ x.float()
    dead = torch.diag(H) == 0
    H[dead, dead] = 1.0
    W[:, dead] = 0
    H += damp * torch.diag(H).mean() * torch.eye(n_in, device=W.device)
    Hinv = torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(H)), upper=True)
    qmax = 2 ** (bits - 1) - 1
    Q = torch.zeros_like(W)
    scale = None
    for b0 in range(0, n_in, block):
        b1 = min(n_in, b0 + block)
        Wb, Eb = W[:, b0:b1].clone(), torch.zeros(W.shape[0], b1 - b0, device=W.device)
        for j in range(b1 - b0):
            col = b0 + j
            if col % group == 0:
                scale = W[:, col: col + group].abs().amax(-1, keepdim=True).clamp_min(1e-12) / qmax
            wc = Wb[:, j]
            qc = (torch.round(wc / scale[:, 0]).clamp(-qmax - 1, qmax)) * scale[:, 0]
            Q[:, col] = qc
            err = (wc - qc) / Hinv[col, col]
            Wb[:, j:] -= err[:, None] * Hinv[col, col:b1][None, :]
            Eb[:, j] = err
        W[:, b1:] -= Eb @ Hinv[b0:b1, b1:]
    return Q.to(w.dtype)


# ---- microscaling formats
_MX = {"mxfp8": ("e4m3", 448.0, 8), "mxfp6": ("e3m2", 28.0, 4), "mxfp4": ("e2m1", 6.0, 2)}
_E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
_E3M2 = torch.tensor(sorted({(1 + m / 4) * 2.0 ** (e - 3) for e in range(1, 8) for m in range(4)} |
                            {m / 4 * 2.0 ** -2 for m in range(4)}))


def _round_to_grid(x, grid):
    g = grid.to(x.device)
    idx = torch.bucketize(x.abs(), (g[1:] + g[:-1]) / 2)
    return g[idx] * x.sign()


class MXFormat:
    """Names of the micro-scaling element formats (reference: interface_bindings/mx_formats.py:37)."""

    MXFP8_E4M3 = "mxfp8_e4m3"
    MXFP8_E5M2 = "mxfp8_e5m2"
    MXFP6_E3M2 = "mxfp6_e3m2"
    MXFP6_E2M3 = "mxfp6_e2m3"
    MXFP4_E2M1 = "mxfp4_e2m1"
    NVFP4_E2M1 = "nvfp4_e2m1"


@dataclass(frozen=True)
class MXFormatSpec:
    """One element format: total bits, exponent / mantissa bits, exponent bias, elements per shared scale (0 = the
    NVFP4 two-level scaling of ``nvfp4_quantize``) and the largest finite magnitude."""

    name: str
    bits: int
    exp_bits: int
    mant_bits: int
    bias: int
    block_size: int
    max_value: float

    @property
    def emax(self) -> int:
        """Exponent of the largest binade, the amount the shared scale is shifted down by."""
        return int(math.floor(math.log2(self.max_value)))

    def grid(self) -> torch.Tensor:
        """Every non-negative finite value of the format, ascending (sub-normals included)."""
        m = 2 ** self.mant_bits
        vals = {k / m * 2.0 ** (1 - self.bias) for k in range(m)}
        vals |= {(1 + k / m) * 2.0 ** (e - self.bias) for e in range(1, 2 ** self.exp_bits) for k in range(m)}
        return torch.tensor(sorted(v for v in vals if v <= self.max_value))


MX_FORMATS = {
    MXFormat.MXFP8_E4M3: MXFormatSpec("mxfp8_e4m3", 8, 4, 3, 7, 32, 448.0),
    MXFormat.MXFP8_E5M2: MXFormatSpec("mxfp8_e5m2", 8, 5, 2, 15, 32, 57344.0),
    MXFormat.MXFP6_E3M2: MXFormatSpec("mxfp6_e3m2", 6, 3, 2, 3, 32, 28.0),
    MXFormat.MXFP6_E2M3: MXFormatSpec("mxfp6_e2m3", 6, 2, 3, 1, 32, 7.5),
    MXFormat.MXFP4_E2M1: MXFormatSpec("mxfp4_e2m1", 4, 2, 1, 1, 32, 6.0),
    MXFormat.NVFP4_E2M1: MXFormatSpec("nvfp4_e2m1", 4, 2, 1, 1, 0, 6.0),
}


def mx_quantize_spec(x, fmt: str = MXFormat.MXFP8_E4M3, block: int = None):
    """``mx_quantize`` for any entry of ``MX_FORMATS`` by name (NVFP4 goes to ``nvfp4_quantize``). The element
    rounding is to the nearest value of the format's grid, ties away from the smaller neighbour's midpoint."""
    spec = MX_FORMATS[fmt]
    if spec.block_size == 0:
        return nvfp4_quantize(x, block or 16)
    block = block or spec.block_size
    g = x.float().reshape(-1, block)
    amax = g.abs().amax(-1, keepdim=True).clamp_min(2.0 ** -126)
    e = torch.floor(torch.log2(amax)) - spec.emax
    s = torch.exp2(e)
    y = _round_to_grid((g / s).clamp(-spec.max_value, spec.max_value), spec.grid())
    return (y * s).reshape(x.shape).to(x.dtype), e.squeeze(-1).to(torch.int8).reshape(*x.shape[:-1], -1)


def mx_quantize(x, fmt="mxfp8", block=32):
    """OCP microscaling: blocks of 32 share one power-of-two (E8M0) scale 2^(floor(log2 amax) - emax_elem).
    Returns (dequantised tensor, scale exponents int8)."""
    name, fmax, emax = _MX[fmt]
    xf = x.float()
    g = xf.reshape(-1, block)
    amax = g.abs().amax(-1, keepdim=True).clamp_min(2.0 ** -126)
    e = torch.floor(torch.log2(amax)) - emax
    s = torch.exp2(e)
    y = (g / s).clamp(-fmax, fmax)
    if name == "e4m3":
        y = y.to(torch.float8_e4m3fn).float()
    else:
        y = _round_to_grid(y, _E2M1 if name == "e2m1" else _E3M2)
    return (y * s).reshape(x.shape).to(x.dtype), e.squeeze(-1).to(torch.int8).reshape(*x.shape[:-1], -1)


def nvfp4_quantize(x, block=16):
    """NVFP4: e2m1 elements, one e4m3 scale per 16 elements and one fp32 tensor scale."""
    xf = x.float()
    tensor_scale = xf.abs().max().clamp_min(1e-12) / (6.0 * 448.0)
    g = xf.reshape(-1, block)
    bs = (g.abs().amax(-1, keepdim=True) / 6.0 / tensor_scale).clamp(2.0 ** -9, 448.0).to(torch.float8_e4m3fn).float()
    y = _round_to_grid((g / (bs * tensor_scale)).clamp(-6, 6), _E2M1)
    return (y * bs * tensor_scale).reshape(x.shape).to(x.dtype), bs.reshape(*x.shape[:-1], -1), tensor_scale

"""Weight quantisation of one linear layer five ways (int8, fp8 e4m3, micro-scaling MXFP4, AWQ and GPTQ at 4 bits) with
the output error each leaves on held-out inputs. For serving, ``quant.quantize_model_(model, "fp8")`` swaps the large
linear layers of a whole model for fp8-weight layers that run the block-scaled tensor-core GEMMs."""
from _common import seed  # first: makes the package importable from a checkout
import torch

import SneppX_ALG as sx
from sneppx.quant import QuantMode, awq_quantize, gptq_quantize, quantize_int8
from sneppx.quant.algorithms import MXFormat, mx_quantize_spec


def rel_err(a, b) -> float:
    return float((a - b).norm() / b.norm())


def main() -> dict:
    g = seed(9)
    w = torch.randn(256, 512, generator=g) / 512 ** 0.5
    # activations as real layers see them: correlated features (a 64-dimensional factor structure plus noise) and a few
    # channels ten times larger than the rest, which is the case AWQ and GPTQ are built for
    channel = 1.0 + 9.0 * (torch.rand(512, generator=g) < 0.05)
    mix = torch.randn(64, 512, generator=g) / 8.0

    def activations(n):
        return (torch.randn(n, 64, generator=g) @ mix + 0.3 * torch.randn(n, 512, generator=g)) * channel

    x, calib = activations(1024), activations(2048)                           # evaluation and (separate) calibration inputs
    y = x @ w.T
    out = {}
    q, s, zp = quantize_int8(w, QuantMode.INT8_SYMMETRIC)
    out["int8"] = rel_err(x @ (q.float() * s).T, y)
    out["fp8_e4m3"] = rel_err(x @ sx.dequantize_fp8_e4m3(sx.quantize_fp8_e4m3(w)).T, y)
    out["mxfp4"] = rel_err(x @ mx_quantize_spec(w, MXFormat.MXFP4_E2M1)[0].T, y)
    grp = w.reshape(256, -1, 128)
    step = grp.abs().amax(-1, keepdim=True) / 7
    rtn4 = (torch.round(grp / step).clamp(-8, 7) * step).reshape(256, 512)
    out["int4_round_to_nearest"] = rel_err(x @ rtn4.T, y)
    w_awq, scale, alpha = awq_quantize(w, calib.abs().mean(0), group=128, bits=4)      # returned in the original weight domain
    out["int4_awq"] = rel_err(x @ w_awq.T, y)
    out["int4_gptq"] = rel_err(x @ gptq_quantize(w, calib, bits=4, group=128).T, y)
    for k, v in out.items():
        print(f"{k:24s} relative output error {v:.4f}")
    return out


if __name__ == "__main__":
    main()

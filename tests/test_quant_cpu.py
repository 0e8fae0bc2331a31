"""Quantisation algorithms: round-trip error bounds, bit-exact fp8, AWQ / GPTQ beat round-to-nearest."""
import torch

from sneppx_alg_b200 import quant as Q


def test_int8_int4_fp8_roundtrip():
    torch.manual_seed(0)
    w = torch.randn(64, 256)
    for mode in (Q.QuantMode.INT8_SYMMETRIC, Q.QuantMode.INT8_ASYMMETRIC, Q.QuantMode.INT8_PER_CHANNEL):
        q, s, z = Q.quantize_int8(w, mode)
        assert (Q.dequantize_int8(q, s, z) - w).abs().max() <= float(s.max()) * 0.51
    p, s = Q.quantize_int4_packed(w)
    assert p.shape == (64, 128) and p.dtype == torch.uint8
    assert (Q.dequantize_int4_packed(p, s) - w).abs().max() <= float(s.max()) * 0.51 + 1e-6
    # fp8: exactly representable values survive, saturation at the format maximum
    vals = torch.tensor([0.0, 1.0, -1.5, 448.0, 1e6, 2.0 ** -9])
    assert torch.equal(Q.fp8_decode(Q.fp8_encode(vals)), torch.tensor([0.0, 1.0, -1.5, 448.0, 448.0, 2.0 ** -9]))
    assert float(Q.fp8_decode(Q.fp8_encode(torch.tensor([1e9]), Q.QuantMode.FP8_E5M2), Q.QuantMode.FP8_E5M2)) == 57344.0
    assert Q.fp8_encode(torch.tensor([1.0])).item() == 0x38 and Q.fp8_encode(torch.tensor([1.0]), Q.QuantMode.FP8_E5M2).item() == 0x3C
    b, s = Q.quantize_fp8(w)
    assert ((Q.fp8_decode(b) * s - w).abs() / w.abs().clamp_min(0.1)).max() < 0.07


def test_awq_and_gptq_reduce_output_error():
    torch.manual_seed(0)
    w = torch.randn(32, 256)
    act = torch.rand(256) * 0.1
    act[:8] = 10.0                                            # a few salient input channels
    x = torch.randn(512, 256) * act
    rtn = Q.dequantize_int4_packed(*Q.quantize_int4_packed(w))
    err_rtn = ((x @ (rtn - w).T) ** 2).mean()
    wq, s, a = Q.awq_quantize(w, x.abs().mean(0))
    assert ((x @ (wq - w).T) ** 2).mean() <= err_rtn
    xg = torch.randn(512, 256) @ torch.randn(256, 256) * 0.1   # correlated inputs: where GPTQ helps
    err_rtn_g = ((xg @ (rtn - w).T) ** 2).mean()
    g = Q.gptq_quantize(w, xg)
    assert ((xg @ (g - w).T) ** 2).mean() < err_rtn_g


def test_mx_and_nvfp4():
    torch.manual_seed(0)
    x = torch.randn(8, 64) * 3
    for fmt, tol in (("mxfp8", 0.13), ("mxfp6", 0.2), ("mxfp4", 0.35)):
        y, e = Q.mx_quantize(x, fmt)
        assert e.shape == (8, 2) and e.dtype == torch.int8
        rel = ((y - x).abs() / x.abs().reshape(-1, 32).amax(-1, keepdim=True).reshape(8, 2).repeat_interleave(32, -1)).max()
        assert rel < tol, (fmt, float(rel))
    y, bs, ts = Q.nvfp4_quantize(x)
    assert bs.shape == (8, 4) and ((y - x).abs().mean() / x.abs().mean()) < 0.15
    # e2m1 grid: every dequantised value / scale is one of the 8 magnitudes
    y4, e4 = Q.mx_quantize(x, "mxfp4")
    mags = (y4.reshape(-1, 32) / torch.exp2(e4.float()).reshape(-1, 1)).abs().unique()
    assert set(mags.tolist()) <= {0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0}


def test_grouped_fp8_reference_and_fp8_moe_on_cpu():
    """CPU statement of the grouped fp8 expert GEMM: close to the unquantised product, zero rows for unused tiles,
    and the MoE layer with fp8 forward GEMMs stays close to the plain layer."""
    import torch

    from sneppx_alg_b200.ops import moe, quant
    torch.manual_seed(0)
    E, N, K = 3, 128, 256
    tg = torch.tensor([2, -1, 0], dtype=torch.int32)
    x = torch.randn(384, K)
    W = torch.randn(E, N, K) * 0.05
    y = quant.gemm_fp8_grouped(x, tg, W)
    assert y[128:256].abs().max() == 0
    full = x[:128] @ W[2].t()
    assert (y[:128] - full).abs().max() / full.abs().max() < 8e-2
    T, d, Fd, k = 64, 128, 128, 2
    xx = torch.randn(T, d)
    idx, w, _, _ = moe.route(torch.randn(T, E), k)
    W1, W2 = torch.randn(E, 2 * Fd, d) * 0.05, torch.randn(E, d, Fd) * 0.05
    a = moe.experts_forward(xx, idx, w, W1, W2, fp8=True)
    b = moe.experts_forward(xx, idx, w, W1, W2)
    assert (a - b).abs().max() / b.abs().max() < 0.1

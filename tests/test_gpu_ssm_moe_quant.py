"""conv1d, chunked SSD scan, router / MoE and quantisation kernels against fp32 PyTorch references."""
import pytest
import torch

from sneppx_alg_b200 import ops
from sneppx_alg_b200.ops import moe, quant, ssm

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)


@pytest.mark.parametrize("with_prev,act", [(False, True), (True, True), (False, False)])
def test_conv1d(with_prev, act):
    torch.manual_seed(0)
    B, L, C, K = 2, 200, 320, 4
    x = torch.randn(B, L, C, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (0.5 * torch.randn(C, K, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    b = torch.randn(C, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    prev = torch.randn(B, K - 1, C, device="cuda", dtype=torch.bfloat16) if with_prev else None
    y = ssm.causal_conv1d(x, w, b, act, prev)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = [t.detach().float().requires_grad_(True) for t in (x, w, b)]
    yr = ssm.conv1d_reference(xr, wr, br, act, prev.float() if with_prev else None)
    yr.backward(g.float())
    assert _rel(y, yr) < 2e-2
    assert _rel(x.grad, xr.grad) < 3e-2 and _rel(w.grad, wr.grad) < 3e-2 and _rel(b.grad, br.grad) < 3e-2


@pytest.mark.parametrize("L,chunk,G", [(256, 64, 1), (512, 256, 2), (200, 64, 1)])
def test_ssd_chunked_vs_recurrence(L, chunk, G):
    torch.manual_seed(0)
    B, H, P, N = 2, 4, 64, 64
    x = torch.randn(B, L, H, P, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    dt = (torch.rand(B, L, H, device="cuda") * 0.1 + 1e-3).requires_grad_(True)
    A = (-torch.rand(H, device="cuda") * 4 - 0.5).requires_grad_(True)
    Bm = torch.randn(B, L, G, N, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    Cm = torch.randn(B, L, G, N, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    D = torch.randn(H, device="cuda", requires_grad=True)
    y = ssm.ssd_scan(x, dt, A, Bm, Cm, D, chunk=chunk)
    g = torch.randn_like(y)
    y.backward(g)
    ops.check_status()
    ref_in = [t.detach().float().requires_grad_(True) for t in (x, dt, A, Bm, Cm, D)]
    yr = ssm.ssd_reference(*ref_in)
    yr.backward(g.float())
    assert _rel(y, yr) < 3e-2
    for got, ref, name in zip((x, dt, A, Bm, Cm, D), ref_in, "x dt A B C D".split()):
        assert _rel(got.grad, ref.grad) < 6e-2, name


def test_conv1d_strided_input_and_gate_mul():
    """conv1d reads a column slice of a wider tensor in place; the output gate y * silu(z) does the same for z."""
    torch.manual_seed(2)
    B, L, C, W = 2, 300, 192, 512
    wide = torch.randn(B, L, W, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(C, 4, device="cuda") * 0.3).to(torch.bfloat16).requires_grad_(True)
    b = torch.randn(C, device="cuda", dtype=torch.bfloat16).requires_grad_(True)
    y = ssm.causal_conv1d(wide[..., 64:64 + C], w, b, act=True)
    out = ssm.gate_mul(y, wide[..., 320:320 + C])
    g = torch.randn_like(out)
    out.backward(g)
    wr, ww, bb = [t.detach().float().requires_grad_(True) for t in (wide, w, b)]
    yr = ssm.conv1d_reference(wr[..., 64:64 + C], ww, bb, True, None)
    outr = yr * torch.nn.functional.silu(wr[..., 320:320 + C])
    outr.backward(g.float())
    assert _rel(out, outr) < 2e-2
    assert _rel(wide.grad, wr.grad) < 3e-2 and _rel(w.grad, ww.grad) < 3e-2 and _rel(b.grad, bb.grad) < 3e-2


def test_ssd_scan_states_and_long_chunks():
    """Initial and final state, their gradients, chunk 128 with 128 state columns (the Mamba-2 2.7B tiling)."""
    torch.manual_seed(1)
    B, L, H, P, N, G = 1, 384, 8, 64, 128, 1
    mk = lambda *s, dt=torch.bfloat16: torch.randn(*s, device="cuda", dtype=dt)
    x = mk(B, L, H, P).requires_grad_(True)
    dt = (torch.rand(B, L, H, device="cuda") * 0.1 + 1e-3).requires_grad_(True)
    A = (-torch.rand(H, device="cuda") * 4 - 0.5).requires_grad_(True)
    Bm, Cm = mk(B, L, G, N).requires_grad_(True), mk(B, L, G, N).requires_grad_(True)
    D = mk(H, dt=torch.float32).requires_grad_(True)
    h0 = mk(B, H, P, N, dt=torch.float32).requires_grad_(True)
    ins = [x, dt, A, Bm, Cm, D, h0]
    y, hf = ssm.ssd_scan(x, dt, A, Bm, Cm, D, chunk=128, init_state=h0, return_state=True)
    g, gf = torch.randn_like(y), torch.randn_like(hf)
    grads = torch.autograd.grad((y.float() * g.float()).sum() + (hf * gf).sum(), ins)
    ops.check_status()
    ref = [t.detach().float().requires_grad_(True) for t in ins]
    yr, hr = ssm.ssd_reference(*ref[:6], init_state=ref[6], return_state=True)
    gr = torch.autograd.grad((yr * g.float()).sum() + (hr * gf).sum(), ref)
    assert _rel(y, yr) < 3e-2 and _rel(hf, hr) < 3e-2
    for got, want, name in zip(grads, gr, "x dt A B C D h0".split()):
        assert _rel(got, want) < 6e-2, name


def test_ssd_fused_chunk_kernel_matches_staged_path(monkeypatch):
    """tcgen05 output-stage kernel (chunk 128, state 128, headdim 64) against the staged path and the fp32 recurrence;
    x, B and C are column slices of one wider token-major tensor, as in the Mamba-2 block; two B/C groups."""
    torch.manual_seed(4)
    B, L, H, P, N, G = 2, 512, 8, 64, 128, 2
    wide = torch.randn(B, L, H * P + 2 * G * N + 64, device="cuda", dtype=torch.bfloat16)
    x = wide[..., :H * P].reshape(B, L, H, P)
    Bm = wide[..., H * P:H * P + G * N].reshape(B, L, G, N)
    Cm = wide[..., H * P + G * N:H * P + 2 * G * N].reshape(B, L, G, N)
    dt = torch.rand(B, L, H, device="cuda") * 0.1 + 1e-3
    A = -torch.rand(H, device="cuda") * 4 - 0.5
    D = torch.randn(H, device="cuda")
    h0 = torch.randn(B, H, P, N, device="cuda")
    with torch.no_grad():
        y1, f1 = ssm.ssd_scan(x, dt, A, Bm, Cm, D, chunk=128, init_state=h0, return_state=True)
        ops.check_status()
        monkeypatch.setenv("SX_SSD_FUSED", "0")
        y0, f0 = ssm.ssd_scan(x, dt, A, Bm, Cm, D, chunk=128, init_state=h0, return_state=True)
        yr = ssm.ssd_reference(x.float(), dt, A, Bm.float(), Cm.float(), D, init_state=h0)
    assert _rel(y1, yr) < 2e-2 and _rel(y0, yr) < 2e-2
    assert _rel(y1, y0) < 1e-2 and torch.equal(f1, f0)


def test_router_and_moe_layer():
    torch.manual_seed(0)
    T, d, E, k, Fd = 1000, 256, 16, 4, 192
    x = torch.randn(T, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    logits = torch.randn(T, E, device="cuda")
    idx, w, probs, counts = moe.route(logits, k)
    ref_idx = moe.topk_reference(torch.softmax(logits, -1), k)
    assert torch.equal(idx.sort(-1).values, ref_idx.sort(-1).values)
    assert torch.allclose(w.sum(-1), torch.ones(T, device="cuda"), atol=1e-5)
    assert counts.sum().item() == T * k
    W1 = (0.05 * torch.randn(E, 2 * Fd, d, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    W2 = (0.05 * torch.randn(E, d, Fd, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    w = w.detach().requires_grad_(True)
    y = moe.experts_forward(x, idx, w, W1, W2)
    g = torch.randn_like(y)
    y.backward(g)
    ops.check_status()
    xr, wr, W1r, W2r = [t.detach().float().requires_grad_(True) for t in (x, w, W1, W2)]
    yr = moe.moe_reference(xr, idx, wr, W1r, W2r)
    yr.backward(g.float())
    assert _rel(y, yr) < 3e-2
    assert _rel(x.grad, xr.grad) < 4e-2 and _rel(w.grad, wr.grad) < 4e-2
    assert _rel(W1.grad, W1r.grad) < 4e-2 and _rel(W2.grad, W2r.grad) < 4e-2


def test_quant_roundtrip_and_reference():
    torch.manual_seed(0)
    x = torch.randn(300, 512, device="cuda", dtype=torch.bfloat16) * 3
    q, s = quant.quant_fp8_1x128(x)
    qr, sr = quant.quant_fp8_1x128_reference(x)
    assert torch.allclose(s, sr, rtol=1e-6)
    assert (q.float() - qr.float()).abs().max().item() <= 32.0  # at most one e4m3 step at the top binade
    assert (q.view(torch.uint8) != qr.view(torch.uint8)).float().mean().item() < 0.01
    assert _rel(quant.dequant_fp8(q, s, "1x128"), x) < 0.07
    w = torch.randn(200, 384, device="cuda", dtype=torch.bfloat16)
    qw, sw = quant.quant_fp8_128x128(w)
    qwr, swr = quant.quant_fp8_128x128_reference(w)
    assert torch.allclose(sw, swr, rtol=1e-6)
    assert _rel(quant.dequant_fp8(qw, sw, "128x128"), w) < 0.07
    w4 = torch.randn(128, 256, device="cuda", dtype=torch.bfloat16)
    p, s4 = quant.quant_int4(w4)
    pr, s4r = quant.quant_int4_reference(w4)
    assert torch.allclose(s4, s4r, rtol=1e-6) and (p != pr).float().mean().item() < 0.01
    assert _rel(quant.dequant_int4(p, s4), w4) < 0.2


def test_models_train_on_gpu():
    from sneppx_alg_b200.models import ModelConfig, build_model
    from sneppx_alg_b200.training.engine import TrainEngine
    torch.manual_seed(0)
    cfgs = [
        ModelConfig(architecture="mamba2", hidden_size=256, num_hidden_layers=2, vocab_size=1000, ssm_state_size=64,
                    ssm_head_dim=64, ssm_ngroups=1, ssm_chunk_size=64, tie_word_embeddings=True),
        ModelConfig(architecture="hss_ser", hidden_size=256, num_hidden_layers=2, vocab_size=1024, ssm_state_size=64,
                    ssm_head_dim=64, ssm_chunk_size=64, num_experts=8, num_experts_per_token=2,
                    moe_intermediate_size=256, router_aux_loss_coef=0.01, tie_word_embeddings=True),
        ModelConfig(architecture="deepseek_moe", hidden_size=256, num_hidden_layers=2, num_attention_heads=2,
                    head_dim=128, intermediate_size=512, vocab_size=1024, num_experts=8, num_experts_per_token=2,
                    num_shared_experts=1, moe_intermediate_size=128, first_dense_layers=1,
                    router_aux_loss_coef=0.001, max_position_embeddings=256),
    ]
    for cfg in cfgs:
        model = build_model(cfg, dtype=torch.bfloat16, device="cuda")
        eng = TrainEngine(model, lr=2e-3, max_grad_norm=1.0)
        ids = torch.randint(0, 1000, (2, 256), device="cuda")
        first = eng.step(ids, ids).item()
        for _ in range(6):
            last = eng.step(ids, ids).item()
        ops.check_status()
        assert last == last and last < first, (cfg.architecture, first, last)


def test_gemm_fp8_block_scaled():
    """fp8 x fp8 tensor-core GEMM against the fp32 product of the dequantised operands (same quantised inputs, so
    the only differences are accumulation order and the bf16 output rounding)."""
    from sneppx_alg_b200.ops import quant
    torch.manual_seed(0)
    for M, N, K in ((5, 256, 512), (64, 384, 1024), (33, 1000, 256), (200, 128, 2048), (16, 4096, 4096)):
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
        bias = torch.randn(N, device="cuda")
        wq, sw = quant.quant_fp8_128x128(w)
        xq, sx = quant.quant_fp8_1x128(x)
        y = quant.gemm_fp8(None, wq, sw, bias=bias, xq=xq, sx=sx)
        ref = quant.gemm_fp8_reference(xq, sx, wq, sw, bias, torch.float32)
        err = (y.float() - ref).abs().max() / ref.abs().max()
        assert err < 1e-2, (M, N, K, float(err))
        # end to end against the unquantised product: fp8 quantisation noise only
        y2 = quant.gemm_fp8(x, wq, sw, bias=bias)
        full = x.float() @ w.float().t() + bias
        assert (y2.float() - full).abs().max() / full.abs().max() < 8e-2
    from sneppx_alg_b200 import ops
    ops.check_status()


@pytest.mark.parametrize("mode", ["fp8", "int4"])
@pytest.mark.parametrize("rows", [64, 300, 2048])
def test_quantized_linear_all_input_sizes(mode, rows):
    """Decode-size inputs take the fp8 x fp8 / in-GEMM dequant paths, prefill-size inputs expand the weight once and
    use the bf16 GEMM; all must agree with the dequantised-weight product."""
    torch.manual_seed(0)
    lin = torch.nn.Linear(512, 384, bias=True, device="cuda", dtype=torch.bfloat16)
    ql = quant.QuantizedLinear.from_linear(lin, mode)
    x = torch.randn(2, rows // 2, 512, device="cuda", dtype=torch.bfloat16)
    y = ql(x)
    if mode == "fp8":
        w = quant.dequant_fp8(ql.qweight.view(torch.float8_e4m3fn), ql.scales, "128x128", torch.float32)
    else:
        w = quant.dequant_int4(ql.qweight, ql.scales, torch.float32)
    ref = x.float() @ w.t() + lin.bias.float()
    assert y.shape == (2, rows // 2, 384)
    # the fp8 x fp8 path also rounds the activations to e4m3 (3 mantissa bits)
    assert _rel(y, ref) < (6e-2 if (mode == "fp8" and rows <= 256) else 2e-2)


def test_grouped_fp8_expert_gemm_and_fp8_moe_layer():
    """Grouped block-scaled fp8 GEMM (expert-sorted rows x stacked expert matrices) against the fp32 product of the
    de-quantised operands; then the SER layer with fp8 forward expert GEMMs against the fp32 dense oracle."""
    from sneppx_alg_b200.ops import quant
    torch.manual_seed(0)
    E, N, K = 5, 384, 512
    groups = [0, 0, 3, -1, 4, 1, 1, 1, -1]
    tg = torch.tensor(groups, dtype=torch.int32, device="cuda")
    rows = 128 * len(groups)
    x = torch.randn(rows, K, device="cuda", dtype=torch.bfloat16)
    W = (torch.randn(E, N, K, device="cuda") * 0.05).to(torch.bfloat16)
    y = quant.gemm_fp8_grouped(x, tg, W)
    ref = quant.gemm_fp8_grouped_reference(x.float(), tg, W.float())
    assert (y.float() - ref.float()).abs().max() / ref.float().abs().max() < 1e-2
    for t, e in enumerate(groups):       # unused tiles are zero, used ones are not
        blk = y[t * 128:(t + 1) * 128].float().abs().max().item()
        assert (blk == 0.0) == (e < 0)
    ops.check_status()
    T, d, Ex, k, Fd = 1000, 256, 8, 2, 128
    xx = torch.randn(T, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    idx, w, _, _ = moe.route(torch.randn(T, Ex, device="cuda"), k)
    W1 = (0.05 * torch.randn(Ex, 2 * Fd, d, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    W2 = (0.05 * torch.randn(Ex, d, Fd, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    w = w.detach().requires_grad_(True)
    yy = moe.experts_forward(xx, idx, w, W1, W2, fp8=True)
    g = torch.randn_like(yy)
    yy.backward(g)
    ops.check_status()
    xr, wr, W1r, W2r = [t.detach().float().requires_grad_(True) for t in (xx, w, W1, W2)]
    yr = moe.moe_reference(xr, idx, wr, W1r, W2r)
    yr.backward(g.float())
    assert _rel(yy, yr) < 8e-2                       # e4m3 rounding of both operands of both GEMMs
    assert _rel(xx.grad, xr.grad) < 8e-2 and _rel(W1.grad, W1r.grad) < 8e-2 and _rel(W2.grad, W2r.grad) < 8e-2

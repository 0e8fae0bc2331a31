"""RNG, dropout, LayerNorm backward, gradient compression and adversarial-step kernels against PyTorch fp32
restatements of the same ops."""
import pytest
import torch
import torch.nn.functional as F

from sneppx_alg_b200.ops import aux
from sneppx_alg_b200.ops import functional as F_

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [4, 1001, 1 << 20])
def test_rng_fill_matches_counter_oracle(n):
    for mode, a, b, tol in (("uniform", -2.0, 5.0, 1e-5), ("normal", 1.0, 3.0, 5e-3), ("bernoulli", 0.37, 0.0, 0.0)):
        got = aux.rng_fill(n, mode, a, b, seed=0x1234567890ABCDEF, offset=9)
        ref = aux.rng_reference(n, mode, a, b, 0x1234567890ABCDEF, 9, device="cuda")
        assert got.shape == (n,) and (got - ref).abs().max().item() <= tol
    big = aux.rng_fill(1 << 20, "normal", 0.0, 1.0, seed=1)
    assert abs(big.mean().item()) < 5e-3 and abs(big.std().item() - 1.0) < 5e-3


def test_dropout_forward_backward_share_the_mask():
    x = torch.randn(64, 4096, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = aux.dropout(x, 0.1, seed=42, offset=3)
    ref = aux.dropout_reference(x.detach(), 0.1, 42, 3)
    assert torch.equal(y, ref)
    g = torch.randn_like(y)
    y.backward(g)
    assert torch.equal(x.grad, aux.dropout_reference(g, 0.1, 42, 3))
    frac = (y == 0).float().mean().item()
    assert 0.09 < frac < 0.11


@pytest.mark.parametrize("rows,cols", [(7, 64), (300, 768), (1024, 4096), (33, 8192), (5, 8200)])
def test_layernorm_backward(rows, cols):
    torch.manual_seed(1)
    x = (torch.randn(rows, cols, device="cuda") * 2 + 0.5).to(torch.bfloat16).requires_grad_(True)
    w = (1 + 0.1 * torch.randn(cols, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    b = (0.1 * torch.randn(cols, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    g = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
    y = F_.layernorm(x, w, b, 1e-5)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yr = F.layer_norm(xr, (cols,), wr, br, 1e-5)
    yr.backward(g.float())

    def rel(a, r):
        return (a.float() - r).abs().max().item() / (r.abs().max().item() + 1e-6)

    assert rel(y, yr) < 1e-2 and rel(x.grad, xr.grad) < 1.5e-2
    assert rel(w.grad, wr.grad) < 1.5e-2 and rel(b.grad, br.grad) < 1.5e-2


def test_gradient_compression_kernels():
    torch.manual_seed(2)
    x = torch.randn(1 << 16, device="cuda") * torch.rand(1 << 16, device="cuda").exp()
    x[512:768] = 0
    q, s = aux.quant_int8(x)
    qr, sr = aux.quant_int8_reference(x)
    assert torch.allclose(s, sr, rtol=1e-6) and (q.int() - qr.int()).abs().max().item() <= 1
    assert (aux.dequant_int8(q, s) - x).abs().max().item() <= s.max().item() * 0.51
    x[64:96] = 1.0  # ties: lowest indices win
    kept, res = aux.block_top2(x)
    kr, rr = aux.block_top2_reference(x)
    assert torch.equal(kept, kr) and torch.equal(res, rr)
    ts = [torch.randn(4096, device="cuda") for _ in range(5)]
    ws = [0.1, 0.2, 0.3, 0.15, 0.25]
    assert torch.allclose(aux.weighted_average(ts, ws), sum(w * t for w, t in zip(ws, ts)), atol=1e-6)


def test_arc_step_kernels():
    torch.manual_seed(3)
    x0 = torch.rand(8192, device="cuda")
    g = torch.randn(8192, device="cuda")
    g[:16] = 0
    adv = aux.arc_step("fgsm", x0, g, eps=0.03)
    assert torch.allclose(adv, aux.arc_step_reference("fgsm", x0, g, eps=0.03), atol=1e-7)
    nxt = aux.arc_step("pgd", adv, g, x0, eps=0.05, alpha=0.03)
    assert torch.allclose(nxt, aux.arc_step_reference("pgd", adv, g, x0, eps=0.05, alpha=0.03), atol=1e-7)
    assert (nxt - x0).abs().max().item() <= 0.05 + 1e-6
    ob = aux.arc_step("obfuscate", g, eps=0.01)
    assert torch.allclose(ob, aux.arc_step_reference("obfuscate", g, eps=0.01), atol=1e-4)
    sm = aux.arc_step("smooth", x0, eps=0.25, seed=9, offset=1)
    assert torch.allclose(sm, aux.arc_step_reference("smooth", x0, eps=0.25, seed=9, offset=1), atol=2e-3)



def test_debug_bounds_mode_catches_bad_indices_without_faulting():
    """Debug-bounds mode: an out-of-range index is reported by the checking kernel (nothing faults, the context stays
    usable), poisoned outputs come back fully written, and a clean run records nothing."""
    from sneppx_alg_b200.ops import debug, moe
    from sneppx_alg_b200.ops.gemm import gemm as gemm_fn
    debug.enable(True)
    try:
        assert debug.read_record() is None
        torch.manual_seed(0)
        # clean run through the MoE plan / grouped GEMM / paged path: no record, no NaN left in outputs
        T, d, E, k, Fd = 300, 128, 4, 2, 64
        x = torch.randn(T, d, device="cuda", dtype=torch.bfloat16)
        idx, w, _, _ = moe.route(torch.randn(T, E, device="cuda"), k)
        W1 = (0.05 * torch.randn(E, 2 * Fd, d, device="cuda")).to(torch.bfloat16)
        W2 = (0.05 * torch.randn(E, d, Fd, device="cuda")).to(torch.bfloat16)
        y = moe.experts_forward(x, idx, w, W1, W2)
        a = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(192, 128, device="cuda", dtype=torch.bfloat16)
        c = gemm_fn(a, b)
        debug.check()
        assert not torch.isnan(y.float()).any() and not torch.isnan(c.float()).any()
        # a bad expert index is caught before any kernel indexes with it
        bad = idx.clone()
        bad[7, 1] = E + 3
        debug.check_indices(bad, 0, E, debug.SITE_TILE_GROUP)
        with pytest.raises(debug.KernelBoundsError, match="element 15 is 7"):
            debug.check()
        assert debug.read_record() is None                     # cleared; the context still works
        tgt = torch.randint(0, 50, (64,), device="cuda")
        tgt[3] = -100
        debug.check_indices(tgt, 0, 50, debug.SITE_CE_TARGET, also_ok=-100)
        debug.check()
        tgt[5] = 50
        debug.check_indices(tgt, 0, 50, debug.SITE_CE_TARGET, also_ok=-100)
        with pytest.raises(debug.KernelBoundsError, match="cross-entropy target"):
            debug.check()
        p = torch.empty(1000, device="cuda", dtype=torch.bfloat16)
        debug.poison_(p)
        assert torch.isnan(p.float()).all()
        assert float((a.float() @ b.float().t()).sum()) == float((a.float() @ b.float().t()).sum())
    finally:
        debug.enable(False)

"""Bandwidth-bound kernels and attention against fp32 PyTorch references of the same ops."""
import math

import pytest
import torch

from sneppx_alg_b200 import ops
from sneppx_alg_b200.ops import functional as F_
from sneppx_alg_b200.optim.fused import adamw_flat_, adamw_reference, grad_norm_

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("per_head", [False, True])
def test_block_sparse_attention_tile_mask(causal, per_head):
    """Tile-level mask in the forward kernel: random masks (some query tiles with no visible tile at all, some steps
    masked for one of the two query tiles of a CTA only), shared or per head, ragged sequence ends."""
    from sneppx_alg_b200.ops.functional import block_sparse_attention, block_sparse_attention_reference
    torch.manual_seed(3)
    B, Sq, Skv, Hq, Hk, D = 2, 1000, 1000, 8, 2, 128
    q = torch.randn(B, Sq, Hq, D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B, Skv, Hk, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(B, Skv, Hk, D, device="cuda", dtype=torch.bfloat16)
    nq, nk = (Sq + 127) // 128, (Skv + 127) // 128
    bm = torch.rand(B if per_head else 1, Hq if per_head else 1, nq, nk, device="cuda") < 0.45
    bm[..., 3, :] = False          # a query tile that sees nothing
    bm[..., 0, 0] = True
    out = block_sparse_attention(q, k, v, bm if per_head else bm[0, 0], causal=causal)
    ops.check_status()
    ref = block_sparse_attention_reference(q.float(), k.float(), v.float(), bm, causal=causal)
    assert torch.isfinite(out.float()).all()
    assert _rel(out, ref) < 2e-2
    # an all-true mask is plain attention
    full = torch.ones(nq, nk, dtype=torch.bool, device="cuda")
    assert _rel(block_sparse_attention(q, k, v, full, causal=causal), ops.attention(q, k, v, causal=causal)) < 1e-3


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)


@pytest.mark.parametrize("T,d", [(64, 256), (333, 4096), (17, 1032)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm_fwd_bwd(T, d, with_res):
    torch.manual_seed(0)
    x = torch.randn(T, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(T, d, device="cuda", dtype=torch.bfloat16, requires_grad=True) if with_res else None
    w = (1 + 0.1 * torch.randn(d, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    y, h = F_.rmsnorm(x, w, 1e-5, r)
    gy, gh = torch.randn_like(y), torch.randn_like(y)
    (y * gy).sum().backward() if not with_res else ((y * gy).sum() + (h * gh).sum()).backward()
    xr = x.detach().float().requires_grad_(True)
    rr = r.detach().float().requires_grad_(True) if with_res else None
    wr = w.detach().float().requires_grad_(True)
    hr = xr + rr if with_res else xr
    yr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    ((yr * gy.float()).sum() + ((hr * gh.float()).sum() if with_res else 0)).backward()
    assert _rel(y, yr) < 2e-2
    assert _rel(x.grad, xr.grad) < 3e-2
    assert _rel(w.grad, wr.grad) < 3e-2
    if with_res:
        assert _rel(r.grad, rr.grad) < 3e-2


def test_rope_fwd_bwd():
    torch.manual_seed(0)
    B, S, H, Hk, D = 2, 96, 4, 2, 128
    qkv = torch.randn(B, S, (H + 2 * Hk) * D, device="cuda", dtype=torch.bfloat16)
    cos, sin = F_.rope_tables(S, D, 5e5, "cuda")
    ref = F_.rope_reference(qkv[..., : (H + Hk) * D].reshape(B, S, H + Hk, D), cos, sin).reshape(B, S, -1)
    x = qkv.clone().requires_grad_(True)
    out = F_.rope_qk_(x * 1.0, cos, sin, H + Hk, D)
    assert _rel(out[..., : (H + Hk) * D], ref) < 1e-2
    assert torch.equal(out[..., (H + Hk) * D:], qkv[..., (H + Hk) * D:])
    g = torch.randn_like(out)
    out.backward(g)
    # rotation is orthogonal: the backward of g is the inverse rotation
    gref = F_.rope_reference(g[..., : (H + Hk) * D].reshape(B, S, H + Hk, D), cos, -sin).reshape(B, S, -1)
    assert _rel(x.grad[..., : (H + Hk) * D], gref) < 1e-2


@pytest.mark.parametrize("act", ["silu", "gelu", "relu"])
def test_glu(act):
    torch.manual_seed(0)
    gu = torch.randn(100, 2 * 264, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    h = F_.glu(gu, act)
    g = torch.randn_like(h)
    h.backward(g)
    gr = gu.detach().float().requires_grad_(True)
    hr = F_.glu_reference(gr, act)
    hr.backward(g.float())
    assert _rel(h, hr) < 1e-2 and _rel(gu.grad, gr.grad) < 2e-2


@pytest.mark.parametrize("V", [1000, 32000])
def test_cross_entropy(V):
    torch.manual_seed(0)
    T = 77
    logits = (3 * torch.randn(T, V, device="cuda")).to(torch.bfloat16)
    tgt = torch.randint(0, V, (T,), device="cuda")
    tgt[5] = -100
    lr = logits.detach().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lr, tgt, ignore_index=-100)
    ref.backward()
    lg = logits.clone().requires_grad_(True)
    loss = F_.cross_entropy(lg * 1.0, tgt)
    loss.backward()
    assert abs(loss.item() - ref.item()) < 2e-3 * max(1, abs(ref.item()))
    assert (lg.grad.float() - lr.grad).abs().max().item() < 2e-4


def test_linear_cross_entropy():
    torch.manual_seed(0)
    T, d, V = 300, 256, 1024
    h = torch.randn(T, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (0.05 * torch.randn(V, d, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    tgt = torch.randint(0, V, (T,), device="cuda")
    loss = F_.linear_cross_entropy(h, w, tgt, chunk=128)
    loss.backward()
    hr, wr = h.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(hr @ wr.t(), tgt)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 5e-3
    assert _rel(h.grad, hr.grad) < 3e-2 and _rel(w.grad, wr.grad) < 3e-2


def test_adamw_flat_and_norm():
    torch.manual_seed(0)
    n = 100003
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda").to(torch.bfloat16)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    out, flag = grad_norm_([g], max_norm=1.0)
    nrm = g.float().norm().item()
    assert abs(out[1].item() - nrm) < 1e-3 * nrm and flag.item() == 0
    coef = 1.0 / (nrm + 1e-6)
    for step in (1, 2):
        adamw_flat_(p, m, v, g, p16, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, 1.0, out[2:3])
        adamw_reference(pr, mr, vr, g, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, coef)
    assert (p - pr).abs().max().item() < 1e-5
    assert torch.equal(p16, p.to(torch.bfloat16))


@pytest.mark.parametrize("B,S,H,Hk,D,causal,window", [
    (1, 128, 2, 2, 128, True, 0), (2, 384, 4, 2, 128, True, 0), (1, 200, 2, 1, 128, True, 0),
    (1, 256, 2, 2, 128, False, 0), (1, 512, 2, 2, 128, True, 128), (1, 256, 2, 2, 64, True, 0)])
def test_attention_forward(B, S, H, Hk, D, causal, window):
    torch.manual_seed(0)
    q = torch.randn(B, S, H, D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B, S, Hk, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(B, S, Hk, D, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        o = F_.attention(q, k, v, causal=causal, window=window)
    ops.check_status()
    ref = F_.attention_reference(q.float(), k.float(), v.float(), causal, window)
    assert _rel(o, ref) < 2e-2


@pytest.mark.parametrize("B,S,H,Hk,causal,window", [(1, 128, 2, 2, True, 0), (2, 320, 4, 2, True, 0),
                                                    (1, 256, 2, 1, False, 0), (1, 384, 2, 2, True, 128)])
def test_attention_backward(B, S, H, Hk, causal, window):
    torch.manual_seed(0)
    D = 128
    qkv = torch.randn(B, S, (H + 2 * Hk) * D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    q = qkv[..., : H * D].view(B, S, H, D)
    k = qkv[..., H * D: (H + Hk) * D].view(B, S, Hk, D)
    v = qkv[..., (H + Hk) * D:].view(B, S, Hk, D)
    o = F_.attention(q, k, v, causal=causal, window=window)
    g = torch.randn_like(o)
    o.backward(g)
    ops.check_status()
    r = qkv.detach().float().requires_grad_(True)
    qr = r[..., : H * D].view(B, S, H, D)
    kr = r[..., H * D: (H + Hk) * D].view(B, S, Hk, D)
    vr = r[..., (H + Hk) * D:].view(B, S, Hk, D)
    F_.attention_reference(qr, kr, vr, causal, window).backward(g.float())
    assert _rel(o, F_.attention_reference(qr, kr, vr, causal, window)) < 2e-2
    for name, sl in (("dq", slice(0, H * D)), ("dk", slice(H * D, (H + Hk) * D)), ("dv", slice((H + Hk) * D, None))):
        assert _rel(qkv.grad[..., sl], r.grad[..., sl]) < 3e-2, name


def test_differential_attention():
    torch.manual_seed(0)
    B, S, H, D = 1, 256, 2, 128
    q = torch.randn(B, S, 2 * H, D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B, S, 2 * H, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(B, S, H, D, device="cuda", dtype=torch.bfloat16)
    lam = torch.tensor([0.3, 0.6], device="cuda")
    with torch.no_grad():
        o = F_.differential_attention(q, k, v, lam)
    a = F_.attention_reference(q.float(), k.float(), v.float(), True).view(B, S, H, 2, D)
    ref = a[..., 0, :] - lam.view(1, 1, -1, 1) * a[..., 1, :]
    assert _rel(o, ref) < 3e-2

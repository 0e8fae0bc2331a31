"""Context-parallel attention / SSD / conv1d on `world` CPU ranks (gloo) against the single-process result.
Run by tests/test_context_parallel_cpu.py as ``python mp_cp_check.py <world> <port>`` (spawns its own ranks)."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _run(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from sneppx_alg_b200.ops import functional as F_
    from sneppx_alg_b200.ops import ssm
    from sneppx_alg_b200.parallel import context as cp

    torch.manual_seed(0)
    B, S, Hq, Hk, D = 2, 8 * world, 4, 2, 16
    q, k, v = torch.randn(B, S, Hq, D), torch.randn(B, S, Hk, D), torch.randn(B, S, Hk, D)
    go = torch.randn(B, S, Hq, D)
    qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
    ref = F_.attention_reference(qr, kr, vr, causal=True)
    ref.backward(go)
    Sl = S // world
    sl = slice(rank * Sl, (rank + 1) * Sl)

    # contiguous layout, causal
    ql, kl, vl = (t[:, sl].clone().requires_grad_(True) for t in (q, k, v))
    out = cp.cp_attention(ql, kl, vl, causal=True)
    out.backward(go[:, sl])
    assert torch.allclose(out, ref[:, sl], atol=1e-5), "cp attention forward"
    for g, full in ((ql.grad, qr.grad), (kl.grad, kr.grad), (vl.grad, vr.grad)):
        assert torch.allclose(g, full[:, sl], atol=1e-5), "cp attention backward"

    # zigzag layout
    zz = lambda t: cp.zigzag_split(t, world, rank)
    ql, kl, vl = (zz(t).clone().requires_grad_(True) for t in (q, k, v))
    out = cp.cp_attention(ql, kl, vl, causal=True, layout="zigzag")
    out.backward(zz(go))
    assert torch.allclose(out, zz(ref), atol=1e-5), "zigzag forward"
    assert torch.allclose(kl.grad, zz(kr.grad), atol=1e-5) and torch.allclose(ql.grad, zz(qr.grad), atol=1e-5), "zigzag backward"
    full = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(full, out.detach().contiguous())
    assert torch.allclose(cp.zigzag_merge(full), ref, atol=1e-5)

    # ring forward
    ring = cp.ring_attention_forward(q[:, sl], k[:, sl], v[:, sl], causal=True)
    assert torch.allclose(ring, ref[:, sl].detach(), atol=1e-5), "ring forward"
    ring_nc = cp.ring_attention_forward(q[:, sl], k[:, sl], v[:, sl], causal=False)
    assert torch.allclose(ring_nc, F_.attention_reference(q, k, v, causal=False)[:, sl], atol=1e-5), "ring non-causal"

    # ring attention with its backward pass (dK / dV accumulators travel with the blocks), causal and not
    for causal, (o_ref, grads) in ((True, (ref, (qr.grad, kr.grad, vr.grad))), (False, (None, None))):
        if o_ref is None:
            qn, kn, vn = (t.clone().requires_grad_(True) for t in (q, k, v))
            o_ref = F_.attention_reference(qn, kn, vn, causal=False)
            o_ref.backward(go)
            grads = (qn.grad, kn.grad, vn.grad)
        ql, kl, vl = (t[:, sl].clone().requires_grad_(True) for t in (q, k, v))
        out = cp.ring_attention(ql, kl, vl, causal=causal)
        out.backward(go[:, sl])
        assert torch.allclose(out, o_ref[:, sl].detach(), atol=1e-5), f"ring forward causal={causal}"
        for g, full_g, name in zip((ql.grad, kl.grad, vl.grad), grads, "qkv"):
            assert torch.allclose(g, full_g[:, sl], atol=2e-5), f"ring backward d{name} causal={causal}"

    # SSD scan, both modes, with gradients
    H, P, G, N, L = 4, 8, 2, 8, 16 * world
    x = torch.randn(B, L, H, P)
    dt = torch.rand(B, L, H) * 0.5 + 0.05
    A = -torch.rand(H) - 0.2
    Bm, Cm, Dp = torch.randn(B, L, G, N), torch.randn(B, L, G, N), torch.randn(H)
    gy = torch.randn(B, L, H, P)
    leaves = [t.clone().requires_grad_(True) for t in (x, dt, A, Bm, Cm, Dp)]
    yref = ssm.ssd_reference(*leaves)
    yref.backward(gy)
    Ll = L // world
    ls = slice(rank * Ll, (rank + 1) * Ll)
    for mode in ("parallel", "serial"):
        xl, dtl, Bl, Cl = (t[:, ls].clone().requires_grad_(True) for t in (x, dt, Bm, Cm))
        Al, Dl = A.clone().requires_grad_(True), Dp.clone().requires_grad_(True)
        y = cp.cp_ssd_scan(xl, dtl, Al, Bl, Cl, Dl, chunk=8, mode=mode)
        y.backward(gy[:, ls])
        assert torch.allclose(y, yref[:, ls], atol=2e-4, rtol=1e-3), f"ssd {mode} forward"
        for g, full_g in ((xl.grad, leaves[0].grad), (dtl.grad, leaves[1].grad), (Bl.grad, leaves[3].grad), (Cl.grad, leaves[4].grad)):
            assert torch.allclose(g, full_g[:, ls], atol=5e-4, rtol=2e-3), f"ssd {mode} backward"
        # A and D are replicated: their full gradient is the sum over ranks
        for g, full_g in ((Al.grad, leaves[2].grad), (Dl.grad, leaves[5].grad)):
            g = g.clone()
            dist.all_reduce(g)
            assert torch.allclose(g, full_g, atol=2e-3, rtol=2e-3), f"ssd {mode} replicated-parameter gradient"

    # conv1d with halo
    Cc, K = 6, 4
    xc, wc, bc = torch.randn(B, L, Cc), torch.randn(Cc, K), torch.randn(Cc)
    gc = torch.randn(B, L, Cc)
    xr_ = xc.clone().requires_grad_(True)
    cref = ssm.conv1d_reference(xr_, wc, bc, act=True)
    cref.backward(gc)
    xl = xc[:, ls].clone().requires_grad_(True)
    yc = cp.cp_conv1d(xl, wc, bc, act=True)
    yc.backward(gc[:, ls])
    assert torch.allclose(yc, cref[:, ls], atol=1e-5), "conv halo forward"
    assert torch.allclose(xl.grad, xr_.grad[:, ls], atol=1e-5), "conv halo backward"
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    world, port = int(sys.argv[1]), int(sys.argv[2])
    mp.spawn(_run, args=(world, port), nprocs=world, join=True)
    print("CP_OK")

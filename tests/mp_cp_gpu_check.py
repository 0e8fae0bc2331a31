"""Worker for the multi-GPU context-parallel test (run under torch.distributed.run): all-gather-KV attention
(contiguous and zigzag), ring attention forward and the two-pass SSD scan on the native bf16 kernels, against fp32
PyTorch references of the full sequence."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from sneppx_alg_b200.ops import check_status  # noqa: E402
from sneppx_alg_b200.ops import functional as F_  # noqa: E402
from sneppx_alg_b200.ops import ssm  # noqa: E402
from sneppx_alg_b200.parallel import context as cp  # noqa: E402


def rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(0)  # same full tensors on every rank
    bf = torch.bfloat16
    B, S, Hq, Hk, D = 1, 512 * world, 8, 2, 128
    q, k, v = (torch.randn(B, S, h, D, device=dev).to(bf) for h in (Hq, Hk, Hk))
    go = torch.randn(B, S, Hq, D, device=dev).to(bf)
    qr, kr, vr = (t.float().requires_grad_(True) for t in (q, k, v))
    ref = F_.attention_reference(qr, kr, vr, causal=True)
    ref.backward(go.float())
    Sl = S // world
    sl = slice(rank * Sl, (rank + 1) * Sl)
    worst = 0.0
    ql, kl, vl = (t[:, sl].clone().requires_grad_(True) for t in (q, k, v))
    out = cp.cp_attention(ql, kl, vl, causal=True)
    out.backward(go[:, sl])
    worst = max(worst, rel(out, ref[:, sl]), rel(ql.grad, qr.grad[:, sl]), rel(kl.grad, kr.grad[:, sl]), rel(vl.grad, vr.grad[:, sl]))
    zz = lambda t: cp.zigzag_split(t, world, rank)
    ql, kl, vl = (zz(t).clone().requires_grad_(True) for t in (q, k, v))
    out = cp.cp_attention(ql, kl, vl, causal=True, layout="zigzag")
    out.backward(zz(go))
    worst = max(worst, rel(out, zz(ref)), rel(ql.grad, zz(qr.grad)), rel(kl.grad, zz(kr.grad)), rel(vl.grad, zz(vr.grad)))
    ring = cp.ring_attention_forward(q[:, sl], k[:, sl], v[:, sl], causal=True)
    worst = max(worst, rel(ring, ref[:, sl]))
    ql, kl, vl = (t[:, sl].clone().requires_grad_(True) for t in (q, k, v))
    out = cp.ring_attention(ql, kl, vl, causal=True)       # ring form with its backward pass
    out.backward(go[:, sl])
    worst = max(worst, rel(out, ref[:, sl]), rel(ql.grad, qr.grad[:, sl]), rel(kl.grad, kr.grad[:, sl]), rel(vl.grad, vr.grad[:, sl]))
    assert worst < 3e-2, f"context-parallel attention error {worst}"

    H, P, G, N, L = 8, 64, 2, 128, 512 * world
    x = (torch.randn(B, L, H, P, device=dev) * 0.5).to(bf)
    dt = (torch.rand(B, L, H, device=dev) * 0.1 + 0.01)
    A = -(torch.rand(H, device=dev) + 0.5)
    Bm, Cm = ((torch.randn(B, L, G, N, device=dev) * 0.3).to(bf) for _ in range(2))
    Dp = torch.randn(H, device=dev)
    gy = torch.randn(B, L, H, P, device=dev).to(bf)
    leaves = [x.float().requires_grad_(True), dt.clone().requires_grad_(True), A, Bm.float().requires_grad_(True),
              Cm.float().requires_grad_(True), Dp]
    yref = ssm.ssd_chunked(*leaves, chunk=128)
    yref.backward(gy.float())
    Ll = L // world
    ls = slice(rank * Ll, (rank + 1) * Ll)
    xl, dtl, Bl, Cl = (t[:, ls].clone().requires_grad_(True) for t in (x, dt, Bm, Cm))
    y = cp.cp_ssd_scan(xl, dtl, A, Bl, Cl, Dp, chunk=128)
    y.backward(gy[:, ls])
    e = max(rel(y, yref[:, ls]), rel(xl.grad, leaves[0].grad[:, ls]), rel(dtl.grad, leaves[1].grad[:, ls]),
            rel(Bl.grad, leaves[3].grad[:, ls]), rel(Cl.grad, leaves[4].grad[:, ls]))
    assert e < 4e-2, f"context-parallel SSD error {e}"
    check_status()
    dist.barrier()
    if rank == 0:
        print(f"CP_GPU_OK attention {worst:.4f} ssd {e:.4f}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""Tensor-parallel Mamba-2 block on CPU ranks (gloo) against the unsharded block: outputs, input gradients and every
parameter gradient (compared with the matching slice). ``python mp_tp_mamba_check.py <world> <port>``."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _run(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from sneppx_alg_b200.nn.ssm import Mamba2Block
    from sneppx_alg_b200.parallel.tp import TPContext
    from sneppx_alg_b200.parallel.tp_mamba import TPMamba2Block

    torch.manual_seed(0)
    B, L, d = 2, 16 * world, 32
    full = Mamba2Block(d, d_state=16, d_conv=4, expand=2, headdim=8, ngroups=2 * world, chunk_size=8)
    with torch.no_grad():
        full.norm.weight.uniform_(0.5, 1.5)
        full.conv_bias.uniform_(-0.1, 0.1)
    u = torch.randn(B, L, d, requires_grad=True)
    g = torch.randn(B, L, d)
    res = torch.randn(B, L, d)
    yref = full(u) + res
    yref.backward(g)

    tp = TPContext(fused=False)
    blk = TPMamba2Block.from_full(full, tp)
    T = B * L
    rows = slice(rank * T // world, (rank + 1) * T // world)
    u_s = u.detach().reshape(T, d)[rows].clone().requires_grad_(True)
    y_s = blk(u_s, batch=B, residual=res.reshape(T, d)[rows])
    y_s.backward(g.reshape(T, d)[rows])
    assert torch.allclose(y_s, yref.reshape(T, d)[rows], atol=2e-5), "forward"
    assert torch.allclose(u_s.grad, u.grad.reshape(T, d)[rows], atol=2e-5), "input gradient"

    r, di, gn = rank, full.d_inner, full.ngroups * full.d_state
    sl = lambda base, width: slice(base + r * width, base + (r + 1) * width)  # noqa: E731
    gn_l = blk.g_l * full.d_state
    rows_w = [sl(0, blk.di_l), sl(di, blk.di_l), sl(2 * di, gn_l), sl(2 * di + gn, gn_l), sl(2 * di + 2 * gn, blk.h_l)]
    chans = [sl(0, blk.di_l), sl(di, gn_l), sl(di + gn, gn_l)]
    checks = [("in_proj", blk.in_proj.weight.grad, torch.cat([full.in_proj.weight.grad[s] for s in rows_w])),
              ("conv_weight", blk.conv_weight.grad, torch.cat([full.conv_weight.grad[s] for s in chans])),
              ("conv_bias", blk.conv_bias.grad, torch.cat([full.conv_bias.grad[s] for s in chans])),
              ("dt_bias", blk.dt_bias.grad, full.dt_bias.grad[sl(0, blk.h_l)]),
              ("A_log", blk.A_log.grad, full.A_log.grad[sl(0, blk.h_l)]),
              ("D", blk.D.grad, full.D.grad[sl(0, blk.h_l)]),
              ("norm", blk.norm_weight.grad, full.norm.weight.grad[sl(0, blk.di_l)]),
              ("out_proj", blk.out_proj.weight.grad, full.out_proj.weight.grad[:, sl(0, blk.di_l)])]
    for name, got, want in checks:
        assert torch.allclose(got, want, atol=5e-5, rtol=1e-4), f"{name} gradient: {(got - want).abs().max().item()}"
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    world, port = int(sys.argv[1]), int(sys.argv[2])
    mp.spawn(_run, args=(world, port), nprocs=world, join=True)
    print("TP_MAMBA_OK")

"""Worker for the multi-GPU expert-parallel test (run under torch.distributed.run): the fused dispatch / combine
kernels against the all_to_all library path of the same SER layer, forward and backward."""
import copy
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from sneppx_alg_b200.nn.moe import SERMoE  # noqa: E402
from sneppx_alg_b200.ops import check_status  # noqa: E402
from sneppx_alg_b200.parallel import expert as ep  # noqa: E402


def rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(7 + rank)
    d, F, E, k, T = 256, 192, 8, 2, 1024
    layer = SERMoE(d, F, num_experts=E, top_k=k, num_shared_experts=1, dtype=torch.bfloat16, device=dev,
                   ep_group=dist.group.WORLD, init_std=0.05)
    with torch.no_grad():   # router and shared expert are replicated
        dist.broadcast(layer.router.weight, 0)
        for p in layer.shared.parameters():
            dist.broadcast(p, 0)
    worst = 0.0
    orig = ep.ep_experts_forward
    for it in range(3):
        x = torch.randn(T, d, device=dev, dtype=torch.bfloat16, requires_grad=True)
        g = torch.randn(T, d, device=dev, dtype=torch.bfloat16)
        outs = []
        for fused in (True, False):
            ep_fn = (lambda *a, _f=fused: orig(*a, fused=_f))
            import sneppx_alg_b200.parallel.expert as mod
            mod.ep_experts_forward = ep_fn
            for p in layer.parameters():
                p.grad = None
            xx = x.detach().clone().requires_grad_(True)
            y = layer(xx)
            y.backward(g)
            outs.append((y.detach(), xx.grad, layer.w1.grad.clone(), layer.w2.grad.clone(), layer.router.weight.grad.clone()))
        mod.ep_experts_forward = orig
        for a, b in zip(outs[0], outs[1]):
            worst = max(worst, rel(a, b))
    torch.cuda.synchronize()
    check_status()
    ok = worst < 4e-2
    t = torch.tensor([int(ok)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"ep world {world}: worst rel err fused vs library {worst:.3e} ->", "OK" if t.item() else "MISMATCH")
    dist.destroy_process_group()
    sys.exit(0 if t.item() else 1)


if __name__ == "__main__":
    main()

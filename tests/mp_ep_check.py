"""Worker for the multi-GPU expert-parallel test (run under torch.distributed.run): the fused dispatch / combine
kernels of the SER layer, forward and backward, against an fp32 PyTorch oracle that holds every expert on every rank
(dense loop over experts, autograd), and against the all_to_all library path of the same layer."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from sneppx_alg_b200.nn.moe import SERMoE  # noqa: E402
from sneppx_alg_b200.ops import check_status  # noqa: E402
from sneppx_alg_b200.ops import functional as ops  # noqa: E402
from sneppx_alg_b200.ops import moe as moe_ops  # noqa: E402
from sneppx_alg_b200.parallel import expert as ep  # noqa: E402


def rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)


def gather_experts(w, world):
    parts = [torch.empty_like(w) for _ in range(world)]
    dist.all_gather(parts, w.detach().contiguous())
    return torch.cat(parts).float().requires_grad_(True)


def oracle(layer, x, g, world):
    """fp32: y = shared(x) + sum_r w_r * expert_{idx_r}(x); returns y, dx, dW1 / dW2 (all experts, summed over ranks),
    d(router weight) of this rank's tokens."""
    W1, W2 = gather_experts(layer.w1, world), gather_experts(layer.w2, world)
    Wr = layer.router.weight.detach().float().requires_grad_(True)
    sh = [p.detach().float().requires_grad_(True) for p in (layer.shared.gate_up_proj.weight, layer.shared.down_proj.weight)]
    xf = x.detach().float().requires_grad_(True)
    # the same expert choice as the layer (chosen from its bf16 logits); weights from fp32 logits
    idx, _, _, _ = moe_ops.route(ops.linear(x.detach(), layer.router.weight).float(), layer.k, layer.renorm)
    probs = torch.softmax(xf @ Wr.t(), -1)
    w = probs.gather(1, idx.long())
    w = w / w.sum(-1, keepdim=True)
    y = torch.zeros_like(xf)
    for e in range(W1.shape[0]):
        tok, slot = (idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = xf[tok] @ W1[e].t()
        a, b = h.chunk(2, -1)
        y = y.index_add(0, tok, (torch.nn.functional.silu(a) * b) @ W2[e].t() * w[tok, slot].unsqueeze(1))
    h = xf @ sh[0].t()
    a, b = h.chunk(2, -1)
    y = y + (torch.nn.functional.silu(a) * b) @ sh[1].t()
    y.backward(g.float())
    dist.all_reduce(W1.grad)
    dist.all_reduce(W2.grad)
    return y.detach(), xf.grad, W1.grad, W2.grad, Wr.grad


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(7 + rank)
    d, F, E, k, T = 256, 192, 8, 2, 1024
    layer = SERMoE(d, F, num_experts=E, top_k=k, num_shared_experts=1, dtype=torch.bfloat16, device=dev,
                   ep_group=dist.group.WORLD, init_std=0.05)
    El = E // world
    with torch.no_grad():   # router and shared expert are replicated
        dist.broadcast(layer.router.weight, 0)
        for p in layer.shared.parameters():
            dist.broadcast(p, 0)
        if rank == 0:
            layer.router.weight[0] *= 6.0    # a popular expert: routing is far from balanced, nothing may be dropped
        dist.broadcast(layer.router.weight, 0)
    worst_oracle, worst_lib = 0.0, 0.0
    for it in range(3):
        x = torch.randn(T, d, device=dev, dtype=torch.bfloat16)
        g = torch.randn(T, d, device=dev, dtype=torch.bfloat16)
        outs = []
        for fused in (True, False):
            ep.FORCE_FUSED = fused
            for p in layer.parameters():
                p.grad = None
            xx = x.detach().clone().requires_grad_(True)
            y = layer(xx)
            y.backward(g)
            outs.append((y.detach(), xx.grad, layer.w1.grad.clone(), layer.w2.grad.clone(), layer.router.weight.grad.clone()))
        ep.FORCE_FUSED = None
        for a, b in zip(outs[0], outs[1]):
            worst_lib = max(worst_lib, rel(a, b))
        y_r, dx_r, dW1_r, dW2_r, dWr_r = oracle(layer, x, g, world)
        ref = (y_r, dx_r, dW1_r[rank * El:(rank + 1) * El], dW2_r[rank * El:(rank + 1) * El], dWr_r)
        for a, b in zip(outs[0], ref):
            worst_oracle = max(worst_oracle, rel(a, b))
    torch.cuda.synchronize()
    check_status()
    dropped = ep.dropped_entries()
    ok = worst_oracle < 4e-2 and worst_lib < 4e-2 and dropped == 0
    t = torch.tensor([int(ok)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"ep world {world}: worst rel err fused vs fp32 oracle {worst_oracle:.3e}, vs library {worst_lib:.3e}, "
              f"dropped {dropped} ({ep.policy_name()}) ->", "OK" if t.item() else "MISMATCH")
    dist.destroy_process_group()
    sys.exit(0 if t.item() else 1)


if __name__ == "__main__":
    try:
        main()
    except SystemExit:
        raise
    except BaseException:  # noqa: BLE001  (the launcher only keeps the tail of stderr: put the cause on stdout)
        import traceback
        print("WORKER ERROR on rank", os.environ.get("RANK"), flush=True)
        traceback.print_exc(file=sys.stdout)
        sys.stdout.flush()
        os._exit(1)

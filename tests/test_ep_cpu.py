"""Expert-parallel SER layer on CPU ranks (gloo): the all-to-all library path must equal the single-process layer
that holds all experts, forward and backward."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sneppx_alg_b200.nn.moe import SERMoE


def _make(ep_group=None):
    torch.manual_seed(0)
    full = SERMoE(32, 48, num_experts=4, top_k=2, num_shared_experts=1, aux_loss_coef=0.01)
    return full


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    full = _make()
    torch.manual_seed(0)
    layer = SERMoE(32, 48, num_experts=4, top_k=2, num_shared_experts=1, aux_loss_coef=0.01, ep_group=dist.group.WORLD)
    with torch.no_grad():
        layer.router.weight.copy_(full.router.weight)
        layer.shared.load_state_dict(full.shared.state_dict())
        el = layer.E_local
        layer.w1.copy_(full.w1[rank * el: (rank + 1) * el])
        layer.w2.copy_(full.w2[rank * el: (rank + 1) * el])
    x = torch.randn(24, 32, generator=torch.Generator().manual_seed(10 + rank), requires_grad=True)
    y = layer(x)
    g = torch.randn(24, 32, generator=torch.Generator().manual_seed(20 + rank))
    y.backward(g)
    xr = x.detach().clone().requires_grad_(True)
    yr = full(xr)
    yr.backward(g)
    err = max((y - yr).abs().max().item(), (x.grad - xr.grad).abs().max().item())
    # expert weight grads: the owner accumulates contributions of all ranks' tokens
    gw = full.w1.grad.clone()  # dense replica: grads of ALL experts from this rank's tokens only
    q.put((rank, err, layer.w1.grad.tolist(), gw.tolist()))
    dist.barrier()
    dist.destroy_process_group()


def test_ep_library_path_matches_dense():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29800 + os.getpid() % 1000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(2)]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, err, gw_ep, gw_full_local in res:
        assert err < 1e-4, (rank, err)
    # sum over ranks of the dense layer's local-token grads equals the owner's EP grad
    import torch as _t
    for owner in range(2):
        ep_grad = _t.tensor([a for r, _, a, _ in res if r == owner][0])
        # the dense replicas each saw only their own tokens: their grads for the owner's experts add up to the EP grad
        dense_sum = sum(_t.tensor(b) for _, _, _, b in res)[owner * 2: (owner + 1) * 2]
        assert (ep_grad - dense_sum).abs().max().item() < 1e-4

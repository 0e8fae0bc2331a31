"""Hierarchical all-reduce (2 nodes x 2 ranks) and Ulysses sequence-parallel attention on 4 CPU ranks (gloo) against
flat / single-process results. Run by tests/test_hier_ulysses_cpu.py as ``python mp_hier_ulysses_check.py <port>``."""
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
    from sneppx_alg_b200.parallel import context as cp
    from sneppx_alg_b200.parallel.hierarchical import HierarchicalAllReduce, hierarchical_all_reduce, make_node_groups

    # ---- hierarchical all-reduce: odd sizes, sum and mean, bucketed gradient lists
    intra, inter = make_node_groups(2)
    assert dist.get_world_size(intra) == 2 and dist.get_world_size(inter) == 2
    for n in (1, 7, 64, 1001):
        torch.manual_seed(100 + rank)
        t = torch.randn(n)
        flat = t.clone()
        dist.all_reduce(flat)
        got = hierarchical_all_reduce(t.clone(), intra, inter)
        assert torch.allclose(got, flat, atol=1e-5), ("sum", n)
        mean = hierarchical_all_reduce(t.clone(), intra, inter, average=True)
        assert torch.allclose(mean, flat / world, atol=1e-6), ("mean", n)
    sync = HierarchicalAllReduce(2, bucket_bytes=4096, average=True)
    torch.manual_seed(7 + rank)
    grads = [torch.randn(300), torch.randn(17, 9), torch.randn(2000), torch.randn(5).double()]
    want = []
    for g in grads:
        w = g.clone()
        dist.all_reduce(w)
        want.append(w / world)
    sync.all_reduce(grads)
    assert all(torch.allclose(g, w, atol=1e-6) for g, w in zip(grads, want))
    total = sum(g.numel() * g.element_size() for g in grads)
    assert total / 2 <= sync.bytes_inter_node <= total / 2 + 64          # half of the bytes cross nodes per rank

    # ---- Ulysses attention: forward and backward against the unsharded computation, MHA and grouped KV heads
    for Hq, Hk in ((8, 8), (8, 4), (8, 2)):
        torch.manual_seed(0)
        B, S, D = 2, 8 * world, 16
        q, k, v = torch.randn(B, S, Hq, D), torch.randn(B, S, Hk, D), torch.randn(B, S, Hk, D)
        go = torch.randn(B, S, Hq, D)
        qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
        ref = F_.attention_reference(qr, kr, vr, causal=True)
        ref.backward(go)
        sl = slice(rank * S // world, (rank + 1) * S // world)
        ql, kl, vl = (t[:, sl].clone().requires_grad_(True) for t in (q, k, v))
        out = cp.ulysses_attention(ql, kl, vl, causal=True)
        out.backward(go[:, sl])
        assert torch.allclose(out, ref[:, sl], atol=1e-5), ("ulysses forward", Hq, Hk)
        for g, full in ((ql.grad, qr.grad), (kl.grad, kr.grad), (vl.grad, vr.grad)):
            assert torch.allclose(g, full[:, sl], atol=1e-5), ("ulysses backward", Hq, Hk)
    try:
        cp.ulysses_attention(torch.randn(1, 4, 6, 8), torch.randn(1, 4, 6, 8), torch.randn(1, 4, 6, 8))
        raise AssertionError("6 heads over 4 ranks must be refused")
    except ValueError:
        pass
    dist.barrier()
    if rank == 0:
        print("HIER_ULYSSES_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    mp.spawn(_run, args=(4, int(sys.argv[1])), nprocs=4, join=True)

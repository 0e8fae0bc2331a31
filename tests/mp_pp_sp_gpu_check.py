"""Worker for the 2-GPU run (under torch.distributed.run, NCCL) of the parts that otherwise only run on gloo ranks:
1F1B and interleaved pipeline stages over NCCL p2p, Ulysses sequence-parallel attention (all-to-all of heads) and
the hierarchical all-reduce, each against a single-GPU fp32 PyTorch computation of the same thing."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from sneppx_alg_b200.models import ModelConfig, build_model  # noqa: E402
from sneppx_alg_b200.ops import check_status  # noqa: E402
from sneppx_alg_b200.ops import functional as F_  # noqa: E402
from sneppx_alg_b200.parallel import context as cp  # noqa: E402
from sneppx_alg_b200.parallel.hierarchical import hierarchical_all_reduce, make_node_groups  # noqa: E402
from sneppx_alg_b200.parallel.pipeline import (InterleavedPipelineStage, LlamaStage, PipelineStage, split_layers,  # noqa: E402
                                               split_layers_interleaved)


def rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    assert world == 2
    worst = {}
    # ---- pipeline: bf16 model on the kernels, 2 stages, 4 micro-batches, against the fp32 un-pipelined model
    cfg = ModelConfig(hidden_size=256, num_hidden_layers=4, num_attention_heads=2, num_key_value_heads=1,
                      intermediate_size=512, vocab_size=512, max_position_embeddings=128, rms_norm_eps=1e-5)
    g = torch.Generator().manual_seed(3)
    mbs = [torch.randint(0, 512, (2, 128), generator=g).to(dev) for _ in range(4)]
    torch.manual_seed(0)
    oracle = build_model(cfg, dtype=torch.float32, device=dev)
    total = 0.0
    for ids in mbs:
        loss = oracle(ids, labels=ids)["loss"]
        (loss / 4).backward()
        total += loss.item() / 4
    ref = {n: p.grad for n, p in oracle.named_parameters()}
    for kind in ("1f1b", "interleaved"):
        torch.manual_seed(0)
        model = build_model(cfg, dtype=torch.bfloat16, device=dev)
        if kind == "1f1b":
            rng = split_layers(4, world)[rank]
            stages, ranges = [LlamaStage(model, rng, rank == 0, rank == world - 1)], [rng]
            pipe = PipelineStage(stages[0], hidden_shape=(2, 128, 256), dtype=torch.bfloat16, device=dev)
            loss = pipe.forward_backward(mbs if rank == 0 else None, mbs if rank == world - 1 else None, 4)
        else:
            ranges = split_layers_interleaved(4, world, 2)[rank]
            stages = [LlamaStage(model, r_, first=(c == 0 and rank == 0), last=(c == 1 and rank == world - 1))
                      for c, r_ in enumerate(ranges)]
            pipe = InterleavedPipelineStage(stages, hidden_shape=(2, 128, 256), dtype=torch.bfloat16, device=dev)
            loss = pipe.forward_backward(mbs, mbs, 4)
        e = 0.0
        if rank == world - 1:
            e = abs(float(loss) - total)
        eg = 0.0
        for st, r_ in zip(stages, ranges):
            for n, p in st.named_parameters():
                if n.startswith("layers.") and n.endswith("qkv_proj.weight"):
                    gr = p.grad if p.grad is not None else getattr(p, "main_grad", None)
                    key = f"layers.{r_[int(n.split('.')[1])]}." + n.split(".", 2)[2]
                    eg = max(eg, rel(gr, ref[key]))
        worst[f"pp_{kind}_loss"] = e
        print(f"rank {rank}: pipeline {kind} done", flush=True)
        worst[f"pp_{kind}_grad"] = eg
        dist.barrier()
    # ---- Ulysses attention on the flash-attention kernel
    torch.manual_seed(0)
    B, S, Hq, Hk, D = 1, 512, 8, 4, 128
    q, k, v = (torch.randn(B, S, h, D, device=dev) for h in (Hq, Hk, Hk))
    go = torch.randn(B, S, Hq, D, device=dev)
    qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
    out_ref = F_.attention_reference(qr, kr, vr, causal=True)
    out_ref.backward(go)
    sl = slice(rank * S // world, (rank + 1) * S // world)
    ql, kl, vl = (t[:, sl].to(torch.bfloat16).clone().requires_grad_(True) for t in (q, k, v))
    out = cp.ulysses_attention(ql, kl, vl, causal=True)
    out.backward(go[:, sl].to(torch.bfloat16))
    worst["ulysses_fwd"] = rel(out, out_ref[:, sl])
    worst["ulysses_dq"] = rel(ql.grad, qr.grad[:, sl])
    worst["ulysses_dk"] = rel(kl.grad, kr.grad[:, sl])
    print(f"rank {rank}: ulysses done", flush=True)
    # ---- hierarchical all-reduce (2 "nodes" of 1 rank) on NCCL
    intra, inter = make_node_groups(1)
    torch.manual_seed(100 + rank)
    t = torch.randn(100003, device=dev)
    flat = t.clone()
    dist.all_reduce(flat)
    worst["hier_allreduce"] = rel(hierarchical_all_reduce(t.clone(), intra, inter), flat)
    torch.cuda.synchronize()
    check_status()
    lim = {"pp_1f1b_loss": 3e-2, "pp_interleaved_loss": 3e-2, "hier_allreduce": 1e-5}
    ok = all(v < lim.get(kname, 5e-2) for kname, v in worst.items())
    tt = torch.tensor([int(ok)], device=dev)
    dist.all_reduce(tt, op=dist.ReduceOp.MIN)
    print(f"rank {rank}: " + ", ".join(f"{kname} {v:.2e}" for kname, v in worst.items()), flush=True)
    if rank == 0:
        print("PP_SP_GPU_OK" if tt.item() else "PP_SP_GPU_MISMATCH", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if tt.item() else 1)


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

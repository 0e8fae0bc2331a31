"""Worker for the multi-GPU tensor-parallel Mamba-2 test (run under torch.distributed.run, 2 or 4 GPUs): the
TP = 2 model on the fused all-gather -> GEMM / GEMM -> reduce-scatter kernels against an fp32 PyTorch run of the
unsharded model (loss, gradient of the replicated embedding, gradient of an out_proj shard), then a few steps of the
TP x DP engine."""
import copy
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from sneppx_alg_b200.models import ModelConfig, build_model  # noqa: E402
from sneppx_alg_b200.ops import check_status  # noqa: E402
from sneppx_alg_b200.parallel.tp import TPContext  # noqa: E402
from sneppx_alg_b200.parallel.tp_engine import TPDPEngine, make_tp_dp_groups  # noqa: E402
from sneppx_alg_b200.parallel.tp_mamba import TPMamba2ForCausalLM  # noqa: E402


def rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    tp_group, dp_group, tp_rank, dp_rank = make_tp_dp_groups(2)
    # 16 heads: each rank gets 8 head columns, which keeps the local in_proj width (1160) a multiple of 8 for the GEMMs
    cfg = ModelConfig(architecture="mamba2", hidden_size=512, num_hidden_layers=2, vocab_size=1024, ssm_state_size=64,
                      ssm_conv_kernel=4, ssm_expand=2, ssm_head_dim=64, ssm_ngroups=2, ssm_chunk_size=128,
                      rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=512)
    torch.manual_seed(0)
    full = build_model(cfg, dtype=torch.bfloat16, device=dev)
    oracle = copy.deepcopy(full).float()
    ids = torch.randint(0, 1024, (2, 512), generator=torch.Generator().manual_seed(5 + dp_rank)).to(dev)
    lo = oracle(ids, labels=ids)["loss"]
    lo.backward()
    model = TPMamba2ForCausalLM(copy.deepcopy(full), TPContext(group=tp_group))
    loss = model(ids, labels=ids)["loss"]
    loss.backward()
    model.sync_replicated_grads()
    tot = loss.detach().float().clone()
    dist.all_reduce(tot, group=tp_group)
    e_loss = abs(tot.item() - lo.item())
    e_emb = rel(model.embedding.weight.grad, oracle.embedding.weight.grad)
    di_l = model.mixers[0].di_l
    want = oracle.layers[1].mixer.out_proj.weight.grad[:, tp_rank * di_l:(tp_rank + 1) * di_l]
    e_out = rel(model.mixers[1].out_proj.weight.grad, want)
    # a few optimizer steps through the engine
    model2 = TPMamba2ForCausalLM(copy.deepcopy(full), TPContext(group=tp_group))
    eng = TPDPEngine(model2, tp_group, dp_group, lr=2e-3)
    losses = [float(eng.step(ids, ids)) for _ in range(5)]
    torch.cuda.synchronize()
    check_status()
    ok = e_loss < 3e-2 and e_emb < 5e-2 and e_out < 5e-2 and all(l == l for l in losses) and losses[-1] < losses[0]
    t = torch.tensor([int(ok)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"tp mamba world {world} (tp2 x dp{world // 2}): loss err {e_loss:.3e}, embedding grad rel {e_emb:.3e}, "
              f"out_proj grad rel {e_out:.3e}, engine losses {losses[0]:.3f} -> {losses[-1]:.3f} ->",
              "OK" if t.item() else "MISMATCH")
    dist.barrier()
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

"""ZeRO engine with expert-parallel parameters on two gloo ranks: expert weights stay rank-local (no data-parallel
reduction, local optimizer state), the replicated parameters stay identical across ranks, and the loss falls."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from sneppx_alg_b200.models.config import ModelConfig
    from sneppx_alg_b200.models.deepseek import DeepSeekV2ForCausalLM
    from sneppx_alg_b200.parallel.zero_engine import ZeroEngine
    torch.manual_seed(0)
    cfg = ModelConfig.from_dict(dict(architecture="deepseek_moe", hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                                     num_attention_heads=2, num_key_value_heads=2, head_dim=16, vocab_size=64,
                                     max_position_embeddings=64, num_experts=4, num_experts_per_token=2,
                                     num_shared_experts=1, moe_intermediate_size=32, first_dense_layers=1,
                                     router_aux_loss_coef=0.01))
    model = DeepSeekV2ForCausalLM(cfg, ep_group=dist.group.WORLD)
    with torch.no_grad():                                   # expert weights differ per rank by construction
        for n, p in model.named_parameters():
            if getattr(p, "is_expert", False):
                p.add_(0.01 * (rank + 1))
    eng = ZeroEngine(model, zero_stage=1, lr=1e-2, weight_decay=0.0, max_grad_norm=1.0, fused=False)
    assert eng.efp is not None and len(eng.expert_params) == 2
    g = torch.Generator().manual_seed(5 + rank)
    ids = torch.randint(0, 64, (2, 16), generator=g)
    losses = [float(eng.step(ids, ids)) for _ in range(8)]
    rep = torch.cat([p.detach().reshape(-1) for p in eng.fp.params])
    exp = torch.cat([p.detach().reshape(-1) for p in eng.expert_params])
    q.put((rank, losses, rep.tolist(), exp.tolist()))
    dist.barrier()
    dist.destroy_process_group()


def test_zero_engine_with_expert_parallel_params():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29300 + os.getpid() % 500
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=180) for _ in range(2)])
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    (_, l0, rep0, exp0), (_, l1, rep1, exp1) = res
    assert l0[-1] < l0[0] and l1[-1] < l1[0]
    assert torch.allclose(torch.tensor(rep0), torch.tensor(rep1), atol=1e-6)       # replicated params in sync
    assert not torch.allclose(torch.tensor(exp0), torch.tensor(exp1), atol=1e-4)   # experts are rank-local

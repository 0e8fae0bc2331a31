"""The benchmark's library comparator (PyTorch ops + torch.distributed only) on CPU ranks: every model shape
steps, losses fall, and the expert-parallel / tensor-parallel forms agree with a single rank where they can."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sneppx_alg_b200.benchmarks import library_arm as la
from sneppx_alg_b200.models import ModelConfig


def _cfg(arch):
    if arch == "mamba2":
        return ModelConfig(architecture="mamba2", hidden_size=32, num_hidden_layers=2, vocab_size=128, ssm_state_size=8,
                           ssm_expand=2, ssm_head_dim=8, ssm_ngroups=2, ssm_conv_kernel=4, ssm_chunk_size=8,
                           rms_norm_eps=1e-5, tie_word_embeddings=True)
    if arch == "deepseek_moe":
        return ModelConfig(architecture="deepseek_moe", hidden_size=32, num_hidden_layers=3, num_attention_heads=4,
                           num_key_value_heads=4, intermediate_size=64, vocab_size=128, rms_norm_eps=1e-6,
                           num_experts=8, num_experts_per_token=2, num_shared_experts=1, moe_intermediate_size=16,
                           first_dense_layers=1, router_aux_loss_coef=0.001)
    return ModelConfig(hidden_size=32, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                       intermediate_size=64, vocab_size=128, rms_norm_eps=1e-5)


def _run(arch, world, rank, tp=1, ep=False, steps=6):
    torch.manual_seed(7)
    cfg = _cfg(arch)
    model, eng, par, dp, tp_group = la.build("x", cfg, torch.device("cpu"), world, rank, tp=tp, ep=ep)
    for o in [t[2] for t in eng.opts] + ([eng.e_opt] if eng.e_opt else []):
        for g in o.param_groups:
            g["lr"] = 1e-2
    ids = torch.randint(0, 128, (2, 16), generator=torch.Generator().manual_seed(3))   # one batch, learned by heart
    losses = []
    for _ in range(steps):
        l = eng.step(ids)
        if tp_group is not None:
            l = l.clone()
            dist.all_reduce(l, group=tp_group)
        losses.append(float(l))
    return losses


@pytest.mark.parametrize("arch", ["transformer", "deepseek_moe", "mamba2"])
def test_library_models_train_on_one_rank(arch):
    losses = _run(arch, 1, 0)
    assert all(l == l for l in losses) and losses[-1] < losses[0] - 0.05, losses


def _worker(rank, world, port, arch, tp, ep, q):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q.put((rank, _run(arch, world, rank, tp=tp, ep=ep)))
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.parametrize("arch,tp,ep", [("transformer", 1, False), ("deepseek_moe", 1, True), ("mamba2", 2, False)])
def test_library_models_train_on_two_ranks(arch, tp, ep):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000 + 17 + tp + int(ep)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, arch, tp, ep, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=240) for _ in range(2))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for losses in res.values():
        assert all(l == l for l in losses) and losses[-1] < losses[0] - 0.05, losses
    if arch != "deepseek_moe":
        # every rank sees the same batch and the same initial weights: the two ranks report the same losses
        assert max(abs(a - b) for a, b in zip(res[0], res[1])) < 1e-4
    if arch == "transformer":
        single = _run(arch, 1, 0)
        assert max(abs(a - b) for a, b in zip(res[0], single)) < 1e-3, (res[0], single)

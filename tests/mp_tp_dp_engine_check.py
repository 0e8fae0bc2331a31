"""TP x DP engine on gloo ranks (tp = 2, dp = world / 2) against a single-process step of the unsharded model on the
concatenated batch: loss, updated replicated parameters, replica consistency. ``python mp_tp_dp_engine_check.py <world> <port>``."""
import copy
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _run(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from sneppx_alg_b200.models import ModelConfig, build_model
    from sneppx_alg_b200.parallel.tp import TPContext
    from sneppx_alg_b200.parallel.tp_engine import TPDPEngine, make_tp_dp_groups
    from sneppx_alg_b200.parallel.tp_mamba import TPMamba2ForCausalLM
    from sneppx_alg_b200.training.engine import TrainEngine

    tp = 2
    tp_group, dp_group, tp_rank, dp_rank = make_tp_dp_groups(tp)
    dp = world // tp
    torch.manual_seed(0)
    cfg = ModelConfig(architecture="mamba2", hidden_size=32, num_hidden_layers=2, vocab_size=128, ssm_state_size=16,
                      ssm_conv_kernel=4, ssm_expand=2, ssm_head_dim=8, ssm_ngroups=2, ssm_chunk_size=8, rms_norm_eps=1e-5,
                      tie_word_embeddings=True)
    full = build_model(cfg)
    g = torch.Generator().manual_seed(5)
    batches = [[torch.randint(0, 128, (2, 32), generator=g) for _ in range(dp)] for _ in range(3)]

    ref_model = copy.deepcopy(full)
    ref = TrainEngine(ref_model, lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1, max_grad_norm=1.0)
    ref_losses = [float(ref.step(torch.cat(b), torch.cat(b))) for b in batches]

    model = TPMamba2ForCausalLM(copy.deepcopy(full), TPContext(group=tp_group, fused=False))
    eng = TPDPEngine(model, tp_group, dp_group, lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1, max_grad_norm=1.0)
    losses = []
    for b in batches:
        l = eng.step(b[dp_rank], b[dp_rank])
        dist.all_reduce(l, group=dp_group)
        losses.append(float(l) / dp)
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 2e-4, (losses, ref_losses)
    assert losses[-1] < losses[0]
    # replicated parameters followed the single-process trajectory (AdamW's first steps are sign-like, so compare
    # the fraction of entries that moved differently)
    for name, mine, want in (("embedding", model.embedding.weight, ref_model.embedding.weight), ("final norm", model.norm.weight, ref_model.norm.weight)):
        off = ((mine - want).abs() > 2e-4).float().mean().item()
        assert off < 0.01, (name, off)
    di_l = model.mixers[0].di_l
    want = ref_model.layers[1].mixer.out_proj.weight[:, tp_rank * di_l:(tp_rank + 1) * di_l]
    assert ((model.mixers[1].out_proj.weight - want).abs() > 2e-4).float().mean().item() < 0.01, "sharded out_proj"
    # every rank holds the same replicated values; DP replicas hold the same shards
    flat = eng.fp.flat.clone()
    rep = flat[: eng.rep_end].clone()
    gathered = [torch.empty_like(rep) for _ in range(world)]
    dist.all_gather(gathered, rep)
    assert all(torch.equal(gathered[0], t) for t in gathered), "replicated parameters diverged"
    shard = flat[eng.rep_end:].clone()
    peers = [torch.empty_like(shard) for _ in range(dp)]
    dist.all_gather(peers, shard, group=dp_group)
    assert all(torch.equal(peers[0], t) for t in peers), "data-parallel replicas diverged"
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    world, port = int(sys.argv[1]), int(sys.argv[2])
    mp.spawn(_run, args=(world, port), nprocs=world, join=True)
    print("TP_DP_ENGINE_OK")

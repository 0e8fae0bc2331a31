"""Tensor-parallel Mamba-2 language model on gloo ranks against the unsharded model: loss and the gradients of the
replicated parameters after ``sync_replicated_grads``. ``python mp_tp_mamba_model_check.py <world> <port>``."""
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
    from sneppx_alg_b200.parallel.tp_mamba import TPMamba2ForCausalLM

    torch.manual_seed(0)
    cfg = ModelConfig(architecture="mamba2", hidden_size=32, num_hidden_layers=2, vocab_size=128, ssm_state_size=16,
                      ssm_conv_kernel=4, ssm_expand=2, ssm_head_dim=8, ssm_ngroups=2, ssm_chunk_size=8, rms_norm_eps=1e-5,
                      tie_word_embeddings=True)
    full = build_model(cfg)
    ids = torch.randint(0, 128, (2, 16 * world))
    ref = full(ids, labels=ids)["loss"]
    ref.backward()
    ref_grads = {n: p.grad.clone() for n, p in full.named_parameters()}

    model = TPMamba2ForCausalLM(copy.deepcopy(full), TPContext(fused=False))
    for p in model.parameters():
        p.grad = None
    loss = model(ids, labels=ids)["loss"]
    loss.backward()
    model.sync_replicated_grads()
    total = loss.detach().clone()
    dist.all_reduce(total)
    assert abs(total.item() - ref.item()) < 1e-5, (total.item(), ref.item())
    assert torch.allclose(model.embedding.weight.grad, ref_grads["embedding.weight"], atol=1e-5), "embedding / tied head"
    assert torch.allclose(model.norm.weight.grad, ref_grads["norm.weight"], atol=1e-5), "final norm"
    for i, n in enumerate(model.layer_norms):
        assert torch.allclose(n.weight.grad, ref_grads[f"layers.{i}.norm.weight"], atol=1e-5), f"layer {i} norm"
    di_l = model.mixers[0].di_l
    for i, m in enumerate(model.mixers):
        want = ref_grads[f"layers.{i}.mixer.out_proj.weight"][:, rank * di_l:(rank + 1) * di_l]
        assert torch.allclose(m.out_proj.weight.grad, want, atol=1e-5), f"layer {i} out_proj shard"
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    world, port = int(sys.argv[1]), int(sys.argv[2])
    mp.spawn(_run, args=(world, port), nprocs=world, join=True)
    print("TP_MAMBA_MODEL_OK")

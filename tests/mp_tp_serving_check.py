"""Tensor-parallel serving engine on gloo ranks: every rank must produce exactly the tokens of the single-rank engine,
for requests that join and leave the batch at different steps. ``python mp_tp_serving_check.py <world> <port>``."""
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
    from sneppx_alg_b200.serving.llm_engine import LLMEngine, SamplingParams, TPLlamaPagedRunner
    torch.manual_seed(0)
    cfg = ModelConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=128,
                      vocab_size=160, max_position_embeddings=128, rms_norm_eps=1e-5)
    model = build_model(cfg).eval()
    prompts = [[3, 9, 27, 81, 5], [7, 7], [100, 2, 150, 4, 9, 9, 31, 8, 64], [12]]
    lens = [6, 9, 4, 7]
    ref = LLMEngine(model, num_blocks=64, block_size=4, max_batch_size=2)
    rids = [ref.submit(p, SamplingParams(max_new_tokens=n)) for p, n in zip(prompts, lens)]
    ref.run_until_done()
    want = [ref.finished[i].output for i in rids]
    eng = LLMEngine(model, num_blocks=64, block_size=4, max_batch_size=2, tp_group=dist.group.WORLD)
    assert isinstance(eng.runner, TPLlamaPagedRunner) and eng.runner.H == 4 // world and eng.cache.k[0].shape[-2] == 2 // world
    ids = [eng.submit(p, SamplingParams(max_new_tokens=n)) for p, n in zip(prompts, lens)]
    eng.run_until_done()
    got = [eng.finished[i].output for i in ids]
    assert got == want, (rank, got, want)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    world, port = int(sys.argv[1]), int(sys.argv[2])
    mp.spawn(_run, args=(world, port), nprocs=world, join=True)
    print("TP_SERVING_OK")

"""Mamba-2 training step with tensor parallelism x data parallelism (baseline configuration 4: Mamba-2-2.7B shape,
TP = 2 x DP = 4 on 8 GPUs, seq 8192, micro-batch 1 per DP replica, bf16, AdamW with fp32 master weights).

``python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m sneppx_alg_b200.benchmarks.tp_mamba --tp 2``
``... --model tiny --seq 64 --device cpu`` runs the same code on gloo ranks (used by the tests).

in_proj is all-gather -> GEMM, out_proj GEMM -> reduce-scatter (the fused kernels of ``parallel/tp.py`` on GPUs);
activations between blocks are sequence-parallel. Reports whole-job tokens per second, device-timed, max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--tp", type=int, default=2)
    ap.add_argument("--model", default="mamba2-2.7b")
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    cuda = a.device == "cuda"
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    if not dist.is_initialized():
        dist.init_process_group("nccl" if cuda else "gloo", **({"device_id": dev} if cuda else {}))
    from ..models import ModelConfig, build_model, config_from_name
    from ..parallel.tp import TPContext
    from ..parallel.tp_engine import TPDPEngine, make_tp_dp_groups
    from ..parallel.tp_mamba import TPMamba2ForCausalLM

    tp_group, dp_group, tp_rank, dp_rank = make_tp_dp_groups(a.tp)
    dp = world // a.tp
    if a.model == "tiny":
        cfg = ModelConfig(architecture="mamba2", hidden_size=64, num_hidden_layers=2, vocab_size=256, ssm_state_size=16,
                          ssm_conv_kernel=4, ssm_expand=2, ssm_head_dim=16, ssm_ngroups=2, ssm_chunk_size=16, rms_norm_eps=1e-5,
                          tie_word_embeddings=True)
    else:
        cfg = config_from_name(a.model)
    torch.manual_seed(1234)   # the same unsharded model on every rank, then sharded in place
    full = build_model(cfg, dtype=torch.bfloat16 if cuda else torch.float32, device=dev)
    model = TPMamba2ForCausalLM(full, TPContext(group=tp_group))
    for layer in full.layers:     # the unsharded mixers are no longer needed
        layer.mixer = None
    engine = TPDPEngine(model, tp_group, dp_group, lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, max_grad_norm=1.0)
    gen = torch.Generator().manual_seed(100 + dp_rank)   # TP ranks of one replica see the same batch
    n = a.warmup + a.steps
    batches = [torch.randint(0, cfg.vocab_size, (a.micro_batch, a.seq), generator=gen).to(dev) for _ in range(n)]

    def sync():
        dist.barrier()
        if cuda:
            torch.cuda.synchronize()

    for i in range(a.warmup):
        engine.step(batches[i], batches[i])
    sync()
    if cuda:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    t0 = time.perf_counter()
    loss = None
    for i in range(a.warmup, n):
        loss = engine.step(batches[i], batches[i])
    if cuda:
        e1.record()
    sync()
    ms = e0.elapsed_time(e1) if cuda else (time.perf_counter() - t0) * 1e3
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t)
    tokens = a.micro_batch * a.seq * dp * a.steps
    line = {"metric": "train tokens/sec", "value": tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": world if cuda else 0, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": ms / a.steps, "dtype": "bf16" if cuda else "fp32", "last_loss": float(loss),
            "config": {"model": a.model, "seq_len": a.seq, "global_batch": a.micro_batch * dp, "parallelism": f"tp{a.tp}xdp{dp}",
                       "optimizer": "AdamW b=(0.9,0.95) wd=0.1 fp32 master+moments", "data": "synthetic token ids, random-init weights"}}
    if rank == 0:
        print(json.dumps(line), flush=True)
        if a.out:
            json.dump(line, open(a.out, "w"), indent=1)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

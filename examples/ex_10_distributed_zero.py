"""Data-parallel training with sharded optimizer state (ZeRO) on two ranks. Run directly, it spawns two ``gloo``
processes on this machine; under ``torchrun`` on GPUs (``torchrun --nproc-per-node 8 --master-addr 127.0.0.1
ex_10_distributed_zero.py``) every rank runs ``train`` on its own GPU over NCCL and the fused NVLink kernels."""
from _common import device, seed  # first: makes the package importable from a checkout
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sneppx.models import ModelConfig, build_model
from sneppx.parallel.zero_engine import ZeroEngine


def train(rank: int, world: int, steps: int = 30):
    torch.manual_seed(0)                                    # same initial weights on every rank
    on_gpu = torch.cuda.is_available() and dist.get_backend() == "nccl"
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank))) if on_gpu else torch.device("cpu")
    if on_gpu:                  # the tensor-core kernels want head size 128 and widths that are multiples of 128
        cfg = ModelConfig(hidden_size=512, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                          intermediate_size=1024, vocab_size=4096, max_position_embeddings=256, rms_norm_eps=1e-5)
    else:
        cfg = ModelConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                          intermediate_size=128, vocab_size=256, max_position_embeddings=32, rms_norm_eps=1e-5)
    model = build_model(cfg, dtype=torch.bfloat16 if on_gpu else torch.float32, device=dev)
    engine = ZeroEngine(model, zero_stage=3, lr=1e-2, weight_decay=0.1, max_grad_norm=1.0)
    # every rank trains on its own slice of one task: continue an arithmetic progression modulo the vocabulary size
    g = torch.Generator().manual_seed(100 + rank)
    start, stride = torch.randint(0, 256, (8, 1), generator=g), torch.randint(1, 4, (8, 1), generator=g)
    ids = ((start + stride * torch.arange(17)) % 256).to(dev)
    return [float(engine.step(ids[:, :-1], ids[:, 1:], shift_labels=False)) for _ in range(steps)]


def _spawned(rank: int, world: int, port: int, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    losses = train(rank, world)
    if rank == 0:
        queue.put(losses)
    dist.barrier()
    dist.destroy_process_group()


def main(world: int = 2) -> list:
    if "RANK" in os.environ:                                                  # launched by torchrun
        dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo")
        if torch.cuda.is_available():
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        losses = train(dist.get_rank(), dist.get_world_size())
        if dist.get_rank() == 0:
            print(f"{dist.get_world_size()} ranks: loss {losses[0]:.3f} -> {losses[-1]:.3f}")
        dist.destroy_process_group()
        return losses
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = 29000 + os.getpid() % 3000
    procs = [ctx.Process(target=_spawned, args=(r, world, port, queue)) for r in range(world)]
    for p in procs:
        p.start()
    losses = queue.get(timeout=180)
    for p in procs:
        p.join(60)
    print(f"{world} gloo ranks, ZeRO-3: rank-0 loss {losses[0]:.3f} -> {losses[-1]:.3f}")
    return losses


if __name__ == "__main__":
    main()

"""1F1B pipeline over CPU ranks (gloo): two stages must reproduce the un-pipelined model's loss and gradients."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sneppx_alg_b200.models import ModelConfig, build_model
from sneppx_alg_b200.parallel.pipeline import LlamaStage, PipelineSchedule, PipelineStage, split_layers


def _cfg():
    return ModelConfig(hidden_size=32, num_hidden_layers=4, num_attention_heads=2, num_key_value_heads=1,
                       intermediate_size=64, vocab_size=64, max_position_embeddings=16, rms_norm_eps=1e-5)


def _batches():
    g = torch.Generator().manual_seed(3)
    return [torch.randint(0, 64, (2, 16), generator=g) for _ in range(4)]


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    model = build_model(_cfg())
    ranges = split_layers(4, world)
    stage = LlamaStage(model, ranges[rank], rank == 0, rank == world - 1)
    pipe = PipelineStage(stage, hidden_shape=(2, 16, 32), dtype=torch.float32, device="cpu")
    mbs = _batches()
    loss = pipe.forward_backward(mbs if rank == 0 else None, mbs if rank == world - 1 else None, 4)
    grads = {n: p.grad.abs().sum().item() for n, p in stage.named_parameters() if p.grad is not None}
    q.put((rank, None if loss is None else loss.item(), grads))
    dist.barrier()
    dist.destroy_process_group()


def test_schedule_shapes():
    s = PipelineSchedule.one_f_one_b(0, 4, 8)
    assert [k for k, _ in s].count("F") == 8 and [k for k, _ in s].count("B") == 8
    assert s[:3] == [("F", 0), ("F", 1), ("F", 2)]          # warm-up = stages - stage - 1
    assert PipelineSchedule.one_f_one_b(3, 4, 8)[:2] == [("F", 0), ("B", 0)]
    assert [len(r) for r in split_layers(10, 4)] == [3, 3, 2, 2]


def test_pipeline_matches_full_model():
    torch.manual_seed(0)
    model = build_model(_cfg())
    mbs = _batches()
    total = 0.0
    for ids in mbs:
        loss = model(ids, labels=ids)["loss"]
        (loss / 4).backward()
        total += loss.item() / 4
    ref = {n: p.grad.abs().sum().item() for n, p in model.named_parameters()}
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29900 + os.getpid() % 1000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(2)]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    by = {r: (l, g) for r, l, g in res}
    assert abs(by[1][0] - total) < 1e-5
    # first stage holds embedding + layers 0-1, last stage layers 2-3 + norm
    assert abs(by[0][1]["embedding.weight"] - 0) >= 0
    for n, v in by[0][1].items():
        key = n if n.startswith("embedding") else "layers." + n.split("layers.")[1]
        assert abs(v - ref[key]) < 1e-4 * max(1.0, ref[key]) or n.startswith("embedding")
    for n, v in by[1][1].items():
        if n.startswith("layers."):
            i = int(n.split(".")[1])
            key = f"layers.{i + 2}." + n.split(".", 2)[2]
            assert abs(v - ref[key]) < 1e-4 * max(1.0, ref[key]), n


def _worker_interleaved(rank, world, port, q):
    from sneppx_alg_b200.parallel.pipeline import InterleavedPipelineStage, split_layers_interleaved
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    model = build_model(_cfg())
    chunks_of = split_layers_interleaved(4, world, 2)[rank]                    # 2 ranks x 2 chunks x 1 layer
    chunks = [LlamaStage(model, rng, first=(c == 0 and rank == 0), last=(c == 1 and rank == world - 1))
              for c, rng in enumerate(chunks_of)]
    pipe = InterleavedPipelineStage(chunks, hidden_shape=(2, 16, 32), dtype=torch.float32, device="cpu")
    mbs = _batches()
    loss = pipe.forward_backward(mbs, mbs, 4)
    grads = {}
    for c, (ch, rng) in enumerate(zip(chunks, chunks_of)):
        for n, p in ch.named_parameters():
            if p.grad is not None and n.startswith("layers."):
                grads[f"layers.{rng[int(n.split('.')[1])]}." + n.split(".", 2)[2]] = p.grad.abs().sum().item()
    q.put((rank, None if loss is None else loss.item(), grads))
    dist.barrier()
    dist.destroy_process_group()


def test_interleaved_schedule_properties():
    from sneppx_alg_b200.parallel.pipeline import interleaved_schedule
    for P, v, M in ((2, 2, 4), (4, 2, 8), (3, 3, 6)):
        for r in range(P):
            s = interleaved_schedule(r, P, v, M)
            f = [(c, i) for k, c, i in s if k == "F"]
            b = [(c, i) for k, c, i in s if k == "B"]
            assert sorted(f) == sorted(b) == sorted((c, i) for c in range(v) for i in range(M))
            for c, i in b:  # a backward step never precedes its own forward step
                assert s.index(("B", c, i)) > s.index(("F", c, i))
            # a chunk's forward follows the previous chunk's forward of the same micro-batch
            for c in range(1, v):
                for i in range(M):
                    assert s.index(("F", c, i)) > s.index(("F", c - 1, i))
    # more chunks: deeper warm-up on the first rank (it must fill the longer virtual pipeline)
    assert [k for k, _, _ in interleaved_schedule(0, 2, 2, 4)][:5] == ["F", "F", "F", "F", "F"]


def test_interleaved_pipeline_matches_full_model():
    torch.manual_seed(0)
    model = build_model(_cfg())
    mbs = _batches()
    total = 0.0
    for ids in mbs:
        loss = model(ids, labels=ids)["loss"]
        (loss / 4).backward()
        total += loss.item() / 4
    ref = {n: p.grad.abs().sum().item() for n, p in model.named_parameters()}
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 28900 + os.getpid() % 1000
    procs = [ctx.Process(target=_worker_interleaved, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in range(2)]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    by = {r: (l, g) for r, l, g in res}
    assert by[0][0] is None and abs(by[1][0] - total) < 1e-5
    seen = {}
    for r in (0, 1):
        seen.update(by[r][1])
    assert {int(k.split(".")[1]) for k in seen} == {0, 1, 2, 3}  # rank 0 holds layers 0 and 2, rank 1 layers 1 and 3
    for k, v in seen.items():
        assert abs(v - ref[k]) < 1e-4 * max(1.0, ref[k]), k

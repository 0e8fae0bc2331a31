"""ZeRO engine logic on CPU ranks (gloo): the sharded library path must reproduce the single-process engine
when every rank sees the same batch, for every stage."""
import copy
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sneppx_alg_b200.models import ModelConfig, build_model
from sneppx_alg_b200.parallel.zero_engine import ZeroEngine, partition_range
from sneppx_alg_b200.training.engine import TrainEngine


def _cfg(arch="transformer"):
    if arch == "mamba2":   # many small tensors (per-head scalars, conv taps): bucket sizes need their own padding
        return ModelConfig(architecture="mamba2", hidden_size=64, num_hidden_layers=3, vocab_size=256,
                           ssm_state_size=16, ssm_expand=2, ssm_head_dim=16, ssm_ngroups=1, ssm_conv_kernel=4,
                           ssm_chunk_size=8, max_position_embeddings=32, rms_norm_eps=1e-5, tie_word_embeddings=True)
    return ModelConfig(hidden_size=64, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                       intermediate_size=128, vocab_size=256, max_position_embeddings=32, rms_norm_eps=1e-5)


def _worker(rank, world, port, stage, q, arch="transformer"):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    model = build_model(_cfg(arch))
    eng = ZeroEngine(model, zero_stage=stage, lr=1e-2, weight_decay=0.1, max_grad_norm=1.0)
    losses = []
    for step in range(3):
        ids = torch.randint(0, 256, (2, 16), generator=torch.Generator().manual_seed(step))
        losses.append(eng.step(ids, ids).item())
    if rank == 0:
        q.put((losses, eng.fp.flat.clone(), float(eng.last_norm[1])))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("stage", [1, 3])
def test_zero_matches_single_process(stage):
    torch.manual_seed(0)
    ref = build_model(_cfg())
    eng = TrainEngine(ref, lr=1e-2, weight_decay=0.1, max_grad_norm=1.0)
    ref_losses = []
    for step in range(3):
        ids = torch.randint(0, 256, (2, 16), generator=torch.Generator().manual_seed(step))
        ref_losses.append(eng.step(ids, ids).item())
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000 + stage
    procs = [ctx.Process(target=_worker, args=(r, 2, port, stage, q)) for r in range(2)]
    for p in procs:
        p.start()
    losses, flat, nrm = q.get(timeout=120)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert max(abs(a - b) for a, b in zip(losses, ref_losses)) < 1e-4
    # compare parameter values tensor by tensor (flat layouts differ in padding)
    assert abs(nrm - float(eng.last_norm[1])) < 1e-3 * max(1.0, nrm)


def _slots_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = _cfg()
    cfg.num_hidden_layers = 5
    out = {}
    for slots in (0, 2, 3):
        torch.manual_seed(0)
        model = build_model(cfg)
        eng = ZeroEngine(model, zero_stage=3, lr=1e-2, weight_decay=0.1, max_grad_norm=1.0, param_slots=slots)
        if slots:
            assert eng.fp.flat is None and eng._compact.numel() < eng.fp.total
            # the parameters of layers i and i + slots share memory
            a, b = eng.bucket_params[0][0], eng.bucket_params[slots][0]
            assert a.data_ptr() == b.data_ptr()
        losses = []
        for step in range(4):
            ids = torch.randint(0, 256, (2, 16), generator=torch.Generator().manual_seed(100 * rank + step))
            losses.append(eng.step(ids, ids).item())
        with torch.no_grad():          # a forward pass outside a training step gathers layer by layer on demand
            ev = float(model(torch.arange(16).view(1, 16), labels=torch.arange(16).view(1, 16))["loss"])
        out[slots] = (losses, eng.master.numpy().copy(), eng.m.numpy().copy(), float(eng.last_norm[1]), ev)   # by value
    if rank == 0:
        q.put(out)
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_parameter_slots_match_the_resident_parameter_engine():
    """``param_slots=K``: K rotating layer slots instead of the full gathered parameter buffer. Losses, gradient norm,
    master weights and moments after four steps (different data per rank) equal those of the engine that keeps every
    parameter resident, for K = 2 and 3 over five layers."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000 + 40
    procs = [ctx.Process(target=_slots_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = q.get(timeout=300)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    base = out[0]
    for k in (2, 3):
        losses, master, m, nrm, ev = out[k]
        assert losses == base[0], (k, losses, base[0])
        assert (master == base[1]).all() and (m == base[2]).all() and nrm == base[3] and ev == base[4]


def test_zero_buckets_of_small_tensors_split_evenly():
    """Mamba-2 layers hold tensors of 8 and 512 elements; every bucket must still be a multiple of 64 * world."""
    torch.manual_seed(0)
    ref = build_model(_cfg("mamba2"))
    eng = TrainEngine(ref, lr=1e-2, weight_decay=0.1, max_grad_norm=1.0)
    ref_losses = []
    for step in range(3):
        ids = torch.randint(0, 256, (2, 16), generator=torch.Generator().manual_seed(step))
        ref_losses.append(eng.step(ids, ids).item())
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000 + 7
    procs = [ctx.Process(target=_worker, args=(r, 3, port, 3, q, "mamba2")) for r in range(3)]
    for p in procs:
        p.start()
    losses, flat, nrm = q.get(timeout=180)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert max(abs(a - b) for a, b in zip(losses, ref_losses)) < 1e-4


def test_partition_range_reference_rule():
    # first n % w ranks get one extra element
    assert [partition_range(10, 4, r) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert [partition_range(8, 4, r) for r in range(4)] == [(0, 2), (2, 4), (4, 6), (6, 8)]


def _resume_worker(rank, world, port, ckdir, q):
    """Uninterrupted run of 4 steps against: 2 steps, save through the Trainer, new model + Trainer, resume, 2 steps."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from sneppx_alg_b200.training.config import TrainConfig
    from sneppx_alg_b200.training.trainer import Trainer

    def batch(step):     # ranks see different data, so a resume that mixed up shards would show
        return torch.randint(0, 256, (2, 16), generator=torch.Generator().manual_seed(10 * step + rank))

    def make(seed):
        torch.manual_seed(seed)
        cfg = TrainConfig()
        cfg.optimizer.lr, cfg.training.max_grad_norm = 1e-2, 1.0
        cfg.checkpoint.dir, cfg.checkpoint.save_every, cfg.checkpoint["async"] = ckdir, 1000, False
        cfg.logging.tracker = "none"
        cfg.distributed.zero_stage = 3
        return Trainer(build_model(_cfg()), cfg)

    whole = make(0)
    ref = [float(whole.train_step(batch(s))) for s in range(4)]
    first = make(0)
    got = [float(first.train_step(batch(s))) for s in range(2)]
    path = first.save_checkpoint({"loss": got[-1]})
    assert f"_rank_{rank}" in os.path.basename(path)
    second = make(123)                      # different initial weights: only a real restore can reproduce the run
    state = second.ckpt.load_latest()
    assert state is not None and int(state["shard_rank"]) == rank
    second.load_checkpoint(state)
    got += [float(second.train_step(batch(s))) for s in range(2, 4)]
    # a shard of the other rank is refused
    other = os.path.join(ckdir, os.path.basename(path).replace(f"_rank_{rank}", f"_rank_{1 - rank}"))
    try:
        second.ckpt.load(other, restore_rng=False)
        refused = False
    except ValueError:
        refused = True
    q.put((rank, ref, got, refused))
    dist.barrier()
    dist.destroy_process_group()


def test_zero_resume_restores_parameters_and_keeps_every_shard(tmp_path):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000 + 11
    procs = [ctx.Process(target=_resume_worker, args=(r, 2, port, str(tmp_path), q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in range(2)]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, ref, got, refused in res:
        assert max(abs(a - b) for a, b in zip(ref, got)) < 1e-5, (rank, ref, got)
        assert refused
    files = sorted(os.listdir(tmp_path))
    assert any("_rank_0" in f for f in files) and any("_rank_1" in f for f in files)

"""Trainer / config / checkpoint manager / data pipeline on CPU."""
import os

import torch

from sneppx_alg_b200.checkpoint.manager import CheckpointCoordinator, CheckpointManager, reshard_flat
from sneppx_alg_b200.models import ModelConfig, build_model
from sneppx_alg_b200.training.config import TrainConfig
from sneppx_alg_b200.training.data import DataLoader, DistributedSampler, SyntheticTokenDataset, TensorDataset
from sneppx_alg_b200.training.trainer import Trainer


def test_sampler_disjoint_and_epoch_seeded():
    a = DistributedSampler(10, 2, 0, seed=1).indices()
    b = DistributedSampler(10, 2, 1, seed=1).indices()
    assert sorted(a + b) == list(range(10)) and not set(a) & set(b)
    s = DistributedSampler(10, 2, 0, seed=1)
    s.set_epoch(1)
    assert s.indices() != a


def test_mlp_regression_trainer_loss_decreases(tmp_path):
    torch.manual_seed(0)
    x = torch.randn(256, 8)
    y = x @ torch.randn(8, 2)
    model = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 2))
    cfg = TrainConfig({"training": {"epochs": 30, "loss": "mse", "log_every": 8, "max_grad_norm": 0.0},
                       "optimizer": {"name": "adam", "lr": 1e-2, "weight_decay": 0.0},
                       "logging": {"dir": str(tmp_path / "runs"), "level": "error"}})
    hist = Trainer(model, cfg).fit(DataLoader(TensorDataset(x, y), batch_size=32, shuffle=True, prefetch=0))
    assert hist[-1] < 0.5 * hist[0]


def test_lm_trainer_checkpoint_resume_continues_step(tmp_path):
    def make():
        torch.manual_seed(0)
        cfg = ModelConfig(hidden_size=32, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1,
                          intermediate_size=64, vocab_size=64, max_position_embeddings=16, rms_norm_eps=1e-5)
        return build_model(cfg)
    tc = {"training": {"epochs": 1, "max_steps": 4, "log_every": 1}, "optimizer": {"lr": 1e-2},
          "checkpoint": {"dir": str(tmp_path / "ck"), "save_every": 2, "keep_last": 2, "async": False},
          "logging": {"dir": str(tmp_path / "runs"), "level": "error"}}
    ds = SyntheticTokenDataset(64, 16, length=64)
    t1 = Trainer(make(), TrainConfig(tc))
    h1 = t1.fit(DataLoader(ds, batch_size=2, prefetch=0))
    assert t1.step_count == 4 and sorted(os.listdir(tmp_path / "ck"))[0].startswith("best_")
    tc["training"]["max_steps"] = 6
    t2 = Trainer(make(), TrainConfig(tc))
    t2.fit(DataLoader(ds, batch_size=2, prefetch=0))
    assert t2.step_count == 6                      # resumed at 4, ran 2 more
    # continuing from the checkpoint reproduces an uninterrupted run's parameters
    tc["checkpoint"] = {"dir": str(tmp_path / "ck2"), "save_every": 0}
    t3 = Trainer(make(), TrainConfig(tc))
    t3.fit(DataLoader(ds, batch_size=2, prefetch=0))
    assert len(h1) == 4


def test_checkpoint_manager_keep_best_and_coordinator(tmp_path):
    m = CheckpointManager(str(tmp_path / "m"), keep_last=2, keep_best=1, metric="loss", mode="min")
    for step, loss in ((1, 3.0), (2, 1.0), (3, 2.0)):
        m.save(step, {"w": torch.full((3,), float(step))}, {"state": {"m": torch.ones(2) * step}}, metrics={"loss": loss})
    assert [s for s, _ in m.list_checkpoints()] == [2, 3]
    assert float(m.load_best()["model_state"]["w"][0]) == 2.0
    latest = m.load_latest()
    assert latest["step"] == 3 and float(latest["optimizer_state"]["state"]["m"][0]) == 3.0
    coords = [CheckpointCoordinator(str(tmp_path / "c"), r, 2, keep_last=1, async_save=False) for r in range(2)]
    for step in (5, 6):
        for r, c in enumerate(coords):
            c.save(step, {"shard": torch.arange(4) + 10 * r}, {"zero_stage": 3})
    assert coords[0].latest_complete_step() == 6 and coords[0].steps() == [6]
    t, meta = coords[1].load(6)
    assert meta["rank"] == 1 and meta["world_size"] == 2 and t["shard"][0] == 10
    os.remove(coords[0].path(6, 1))
    assert coords[0].latest_complete_step() is None   # a missing rank file makes the step incomplete
    # ZeRO reshard 2 -> 4 ranks keeps the logical flat vector
    bounds = [(0, 8), (8, 24)]
    full = torch.arange(24.0)
    def shards(world):
        return [torch.cat([full[b0:b1].view(world, -1)[r] for b0, b1 in bounds]) for r in range(world)]
    out = reshard_flat(shards(2), bounds, 4)
    assert all(torch.equal(a, b) for a, b in zip(out, shards(4)))

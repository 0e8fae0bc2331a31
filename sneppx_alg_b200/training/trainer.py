"""``Trainer``: config-driven training loop (``train_step`` / ``fit`` / ``evaluate``) with checkpoint resume, LR
schedule, experiment tracking and profiling, following the reference's ``Trainer`` (interface_bindings/trainer_v3.py:
233-718; C twin kernel/train/trainer.c:114-353). Language models (modules whose forward takes ``labels`` and returns a
dict with ``loss``) train through the flat-buffer / ZeRO engines on the fused kernels; any other ``nn.Module`` trains
through a plain optimizer from the zoo with a loss function (mse / cross_entropy), as the reference's linear / MLP
example configs do. Unlike the reference, resuming restores the step counter (trainer_v3.py:577 resets it to 0)."""
from __future__ import annotations

import time
from typing import Callable, Iterable, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..checkpoint.manager import CheckpointManager
from ..optim.zoo import get_optimizer
from ..utils.observability import Logger, Profiler, make_tracker
from .config import TrainConfig
from .schedulers import get_scheduler

LOSSES = {"mse": lambda out, y: F.mse_loss(out.float(), y.float()),
          "cross_entropy": lambda out, y: F.cross_entropy(out.float().view(-1, out.shape[-1]), y.view(-1))}


def _is_lm(model) -> bool:
    import inspect
    try:
        return "labels" in inspect.signature(model.forward).parameters
    except (TypeError, ValueError):
        return False


class Trainer:
    def __init__(self, model, config: Optional[TrainConfig] = None, loss_fn: Optional[Callable] = None,
                 eval_fn: Optional[Callable] = None):
        self.cfg = config or TrainConfig()
        c = self.cfg
        self.model = model
        self.log = Logger(level=c.logging.level)
        self.profiler = Profiler(use_nvtx=c.profiler.enabled)
        self.tracker = make_tracker(c.logging.tracker, directory=c.logging.dir)
        self.step_count, self.epoch = 0, 0
        self.eval_fn = eval_fn
        torch.manual_seed(c.training.seed)
        self.is_lm = _is_lm(model)
        o = c.optimizer
        if self.is_lm:
            distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
            kw = dict(lr=o.lr, betas=tuple(o.betas), eps=o.eps, weight_decay=o.weight_decay,
                      max_grad_norm=c.training.max_grad_norm)
            if distributed:
                from ..parallel.zero_engine import ZeroEngine
                self.engine = ZeroEngine(model, zero_stage=max(1, c.distributed.zero_stage),
                                         fused=None if c.distributed.fused_collectives else False, **kw)
            else:
                from .engine import TrainEngine
                self.engine = TrainEngine(model, **kw)
            self.optimizer = None
            sched_target = self.engine
        else:
            self.engine = None
            self.optimizer = get_optimizer(o.name, model.parameters(), lr=o.lr, betas=o.betas, eps=o.eps,
                                           weight_decay=o.weight_decay)
            self.loss_fn = loss_fn or LOSSES[c.training.loss]
            sched_target = self.optimizer
        s = c.scheduler
        self.scheduler = get_scheduler(s.name, sched_target, base_lr=o.lr, total_steps=s.total_steps or c.training.max_steps,
                                       warmup_steps=s.warmup_steps, min_lr=s.min_lr)
        ck = c.checkpoint
        # A ZeRO engine's state is this rank's shard: every rank then saves its own file (between barriers) and a
        # resume only accepts a step that every rank wrote.
        sharded = self.engine is not None and getattr(self.engine, "world", 1) > 1
        self.ckpt = CheckpointManager(ck.dir, ck.keep_last, ck.keep_best, ck.metric, ck.mode, ck.format,
                                      async_save=bool(ck.get("async", False)),
                                      rank=self.engine.rank if sharded else 0,
                                      world_size=self.engine.world if sharded else 1,
                                      barrier_fn=(lambda: dist.barrier(self.engine.group)) if sharded else None,
                                      trusted=bool(ck.get("trusted", False))) \
            if ck.save_every or ck.resume_from else None

    # ------------------------------------------------------------------ steps
    def train_step(self, batch) -> float:
        x, y = batch if isinstance(batch, (tuple, list)) else (batch, batch)
        dev = next(self.model.parameters()).device
        x, y = x.to(dev, non_blocking=True), y.to(dev, non_blocking=True)
        with self.profiler.range("train_step"):
            if self.is_lm:
                self.scheduler.step()
                loss = self.engine.step(x, y, shift_labels=False) if self._preshifted(x, y) else self.engine.step(x, y)
            else:
                self.scheduler.step()
                self.optimizer.zero_grad(set_to_none=True)
                loss = self.loss_fn(self.model(x), y)
                loss.backward()
                if self.cfg.training.max_grad_norm > 0:
                    torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.cfg.training.max_grad_norm)
                self.optimizer.step()
        self.step_count += 1
        return loss.detach() if torch.is_tensor(loss) else loss

    @staticmethod
    def _preshifted(x, y):
        return x.data_ptr() != y.data_ptr() and x.shape == y.shape and not torch.equal(x, y)

    @torch.no_grad()
    def evaluate(self, loader: Iterable, max_batches: int = 0) -> dict:
        self.model.eval()
        tot, n = 0.0, 0
        dev = next(self.model.parameters()).device
        for i, batch in enumerate(loader):
            x, y = batch if isinstance(batch, (tuple, list)) else (batch, batch)
            x, y = x.to(dev), y.to(dev)
            if self.is_lm:
                loss = self.model(x, labels=y, shift_labels=not self._preshifted(x, y))["loss"]
            else:
                loss = self.loss_fn(self.model(x), y)
            tot += float(loss)
            n += 1
            if max_batches and i + 1 >= max_batches:
                break
        self.model.train()
        out = {"loss": tot / max(n, 1)}
        if self.eval_fn:
            out.update(self.eval_fn(self.model))
        return out

    # ------------------------------------------------------------------ checkpoint
    def state_dict(self):
        sd = {"step": self.step_count, "epoch": self.epoch, "scheduler": self.scheduler.state_dict()}
        if self.engine is not None:
            sd["engine"] = self.engine.state_dict()
        else:
            sd["model"] = self.model.state_dict()
            sd["optimizer"] = self.optimizer.state_dict()
        return sd

    def save_checkpoint(self, metrics=None):
        if self.engine is not None and hasattr(self.engine, "check_status"):
            self.engine.check_status()      # never write a checkpoint after a device wait gave up
        sd = self.state_dict()
        return self.ckpt.save(self.step_count, sd.get("model") or {}, sd.get("optimizer") or sd.get("engine"),
                              self.epoch, metrics, self.cfg.to_dict(), extra={"scheduler": sd["scheduler"]})

    def load_checkpoint(self, state: dict):
        self.step_count, self.epoch = int(state["step"]), int(state.get("epoch", 0))
        if self.engine is not None:
            self.engine.load_state_dict(state["optimizer_state"])
        else:
            self.model.load_state_dict(state["model_state"])
            self.optimizer.load_state_dict(state["optimizer_state"])
        if state.get("extra") and state["extra"].get("scheduler"):
            self.scheduler.load_state_dict(state["extra"]["scheduler"])

    # ------------------------------------------------------------------ loop
    def fit(self, train_loader: Iterable, eval_loader: Optional[Iterable] = None, max_steps: Optional[int] = None):
        c = self.cfg
        max_steps = max_steps or c.training.max_steps or float("inf")
        if self.ckpt is not None:
            state = self.ckpt.load(c.checkpoint.resume_from) if c.checkpoint.resume_from else self.ckpt.load_latest()
            if state is not None:
                self.load_checkpoint(state)
                self.log.info("resumed", step=self.step_count)
        self.tracker.start_run(params=c.to_dict())
        t0, last_log, history = time.perf_counter(), self.step_count, []
        done = False
        while not done and self.epoch < c.training.epochs:
            if hasattr(getattr(train_loader, "sampler", None), "set_epoch"):
                train_loader.sampler.set_epoch(self.epoch)
            for batch in train_loader:
                loss = self.train_step(batch)
                if c.training.log_every and self.step_count % c.training.log_every == 0:
                    lv = float(loss.detach())
                    dt = time.perf_counter() - t0
                    sps = (self.step_count - last_log) / max(dt, 1e-9)
                    t0, last_log = time.perf_counter(), self.step_count
                    history.append(lv)
                    self.tracker.log_metrics({"loss": lv, "steps_per_s": sps, "lr": self.scheduler.get_lr()}, self.step_count)
                    self.log.info(f"step {self.step_count} loss {lv:.4f} {sps:.2f} steps/s")
                metrics = None
                if eval_loader is not None and c.training.eval_every and self.step_count % c.training.eval_every == 0:
                    metrics = self.evaluate(eval_loader)
                    self.tracker.log_metrics({f"eval_{k}": v for k, v in metrics.items()}, self.step_count)
                if self.ckpt is not None and c.checkpoint.save_every and self.step_count % c.checkpoint.save_every == 0:
                    self.save_checkpoint(metrics or {"loss": float(loss.detach())})
                if self.step_count >= max_steps:
                    done = True
                    break
            else:
                self.epoch += 1
        self.tracker.end_run()
        if self.ckpt is not None:
            self.ckpt.close()
        return history

    def print_profile(self):
        print(self.profiler.report())

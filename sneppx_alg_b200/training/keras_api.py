"""Keras-flavoured and trainer-v2 front ends (the reference's ``keras_api.py``: ``Sequential.compile / fit / evaluate /
predict``; ``trainer_v2.py``: ``UltraTrainer`` with EMA, label smoothing and early stopping).  Both are thin layers
over the same modules, optimizers and fused kernels as ``training.trainer.Trainer``."""
from __future__ import annotations

from typing import Callable, List, Optional

import torch
import torch.nn as tnn

from ..optim.zoo import get_optimizer
from .extras import EMA, EarlyStopping, label_smoothing_ce

_LOSSES = {"mse": tnn.functional.mse_loss, "categorical_crossentropy": tnn.functional.cross_entropy,
           "sparse_categorical_crossentropy": tnn.functional.cross_entropy, "binary_crossentropy":
           tnn.functional.binary_cross_entropy_with_logits, "mae": tnn.functional.l1_loss}


class Sequential(tnn.Sequential):
    def compile(self, optimizer="adam", loss="mse", metrics=(), lr=1e-3, **opt_kw):
        self._opt = get_optimizer(optimizer, self.parameters(), lr=lr, **opt_kw) if isinstance(optimizer, str) else optimizer
        self._loss = _LOSSES[loss] if isinstance(loss, str) else loss
        self._metrics = list(metrics)
        return self

    def fit(self, x, y, epochs=1, batch_size=32, validation_data=None, shuffle=True, verbose=0, callbacks=()):
        history = {"loss": [], "val_loss": []}
        n = x.shape[0]
        for ep in range(epochs):
            self.train()
            perm = torch.randperm(n) if shuffle else torch.arange(n)
            tot = 0.0
            for s in range(0, n, batch_size):
                idx = perm[s: s + batch_size]
                loss = self._loss(self(x[idx]), y[idx])
                self._opt.zero_grad()
                loss.backward()
                self._opt.step()
                tot += float(loss.detach()) * len(idx)
            history["loss"].append(tot / n)
            if validation_data is not None:
                history["val_loss"].append(self.evaluate(*validation_data, batch_size=batch_size))
            stop = False
            for cb in callbacks:
                stop |= bool(cb(ep, history))
            if verbose:
                print(f"epoch {ep + 1}/{epochs} loss {history['loss'][-1]:.4f}")
            if stop:
                break
        return history

    @torch.no_grad()
    def evaluate(self, x, y, batch_size=32):
        self.eval()
        tot = 0.0
        for s in range(0, x.shape[0], batch_size):
            tot += float(self._loss(self(x[s: s + batch_size]), y[s: s + batch_size])) * min(batch_size, x.shape[0] - s)
        return tot / x.shape[0]

    @torch.no_grad()
    def predict(self, x, batch_size=32):
        self.eval()
        return torch.cat([self(x[s: s + batch_size]) for s in range(0, x.shape[0], batch_size)])


class UltraTrainer:
    """Classification / regression trainer with EMA weights, label smoothing, gradient clipping, early stopping."""

    def __init__(self, model, optimizer="adamw", lr=1e-3, label_smoothing=0.0, ema_decay=0.0, max_grad_norm=0.0,
                 patience=0, loss_fn: Optional[Callable] = None, **opt_kw):
        self.model = model
        self.opt = get_optimizer(optimizer, model.parameters(), lr=lr, **opt_kw)
        self.ema = EMA(model, ema_decay) if ema_decay > 0 else None
        self.stopper = EarlyStopping(patience) if patience > 0 else None
        self.max_grad_norm = max_grad_norm
        self.loss_fn = loss_fn or ((lambda o, t: label_smoothing_ce(o, t, label_smoothing)) if label_smoothing > 0
                                   else tnn.functional.cross_entropy)
        self.history: List[dict] = []

    def train_step(self, x, y) -> float:
        self.model.train()
        loss = self.loss_fn(self.model(x), y)
        self.opt.zero_grad()
        loss.backward()
        if self.max_grad_norm > 0:
            torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.max_grad_norm)
        self.opt.step()
        if self.ema is not None:
            self.ema.update(self.model)
        return float(loss.detach())

    @torch.no_grad()
    def evaluate(self, x, y) -> dict:
        self.model.eval()
        out = self.model(x)
        res = {"loss": float(tnn.functional.cross_entropy(out, y)) if out.dim() == 2 and y.dtype == torch.long
               else float(self.loss_fn(out, y))}
        if out.dim() == 2 and y.dtype == torch.long:
            res["accuracy"] = float((out.argmax(-1) == y).float().mean())
        return res

    def fit(self, x, y, epochs=1, batch_size=32, val=None):
        n = x.shape[0]
        for ep in range(epochs):
            perm = torch.randperm(n)
            losses = [self.train_step(x[perm[s: s + batch_size]], y[perm[s: s + batch_size]]) for s in range(0, n, batch_size)]
            rec = {"epoch": ep, "loss": sum(losses) / len(losses)}
            if val is not None:
                rec.update({"val_" + k: v for k, v in self.evaluate(*val).items()})
            self.history.append(rec)
            if self.stopper is not None and val is not None and self.stopper.step(rec["val_loss"]):
                break
        return self.history

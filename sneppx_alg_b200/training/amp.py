"""Mixed precision helpers with the reference's names (interface_bindings/amp.py): ``autocast`` context and a
``GradScaler`` with dynamic loss scaling (needed for fp16; bf16 training runs unscaled)."""
from __future__ import annotations

import contextlib

import torch


@contextlib.contextmanager
def autocast(enabled=True, dtype=torch.bfloat16, device_type=None):
    device_type = device_type or ("cuda" if torch.cuda.is_available() else "cpu")
    with torch.autocast(device_type=device_type, dtype=dtype, enabled=enabled):
        yield


class GradScaler:
    def __init__(self, init_scale=2.0 ** 16, growth_factor=2.0, backoff_factor=0.5, growth_interval=2000, enabled=True):
        self.scale_value, self.growth, self.backoff, self.interval, self.enabled = init_scale, growth_factor, backoff_factor, growth_interval, enabled
        self._good, self._found_inf = 0, False

    def scale(self, loss):
        return loss * self.scale_value if self.enabled else loss

    def unscale_(self, optimizer):
        if not self.enabled:
            return
        inv, found = 1.0 / self.scale_value, False
        for g in optimizer.param_groups:
            for p in g["params"]:
                if p.grad is not None:
                    p.grad.mul_(inv)
                    found = found or not bool(torch.isfinite(p.grad).all())
        self._found_inf = found

    def step(self, optimizer):
        if self.enabled and self._found_inf:
            return None
        return optimizer.step()

    def update(self):
        if not self.enabled:
            return
        if self._found_inf:
            self.scale_value *= self.backoff
            self._good = 0
        else:
            self._good += 1
            if self._good % self.interval == 0:
                self.scale_value *= self.growth
        self._found_inf = False

    def state_dict(self):
        return {"scale": self.scale_value, "good": self._good}

    def load_state_dict(self, sd):
        self.scale_value, self._good = sd["scale"], sd["good"]

"""``TrainConfig``: YAML / JSON training configuration deep-merged over defaults, with ``--override`` JSON patches and
attribute-style section views. Section names and default keys follow the reference
(interface_bindings/trainer_v3.py:38-170: training / optimizer / scheduler / amp / logging / checkpoint /
distributed / profiler / privacy)."""
from __future__ import annotations

import copy
import json
from typing import Any, Dict, Optional

DEFAULTS: Dict[str, Any] = {
    "training": {"epochs": 1, "max_steps": 0, "batch_size": 8, "seq_len": 512, "grad_accum_steps": 1,
                 "max_grad_norm": 1.0, "seed": 0, "loss": "cross_entropy", "eval_every": 0, "log_every": 10},
    "model": {"name": "", "overrides": {}},
    "optimizer": {"name": "adamw", "lr": 1e-3, "betas": [0.9, 0.999], "eps": 1e-8, "weight_decay": 0.01},
    "scheduler": {"name": "constant", "warmup_steps": 0, "min_lr": 0.0, "total_steps": 0},
    "amp": {"enabled": True, "dtype": "bfloat16", "loss_scale": "dynamic"},
    "logging": {"dir": "runs", "tracker": "local", "level": "info"},
    "checkpoint": {"dir": "checkpoints", "save_every": 0, "keep_last": 3, "keep_best": 1, "resume_from": None,
                   "format": "binary", "async": True, "metric": "loss", "mode": "min", "trusted": False},
    "distributed": {"enabled": False, "backend": "nccl", "zero_stage": 0, "tensor_parallel_size": 1,
                    "pipeline_parallel_size": 1, "expert_parallel_size": 1, "num_microbatches": 1,
                    "bucket_size_mb": 25, "overlap_comm": True, "fused_collectives": True},
    "profiler": {"enabled": False, "warmup": 2, "active": 5},
    "privacy": {"enabled": False, "noise_multiplier": 1.0, "max_grad_norm": 1.0, "delta": 1e-5},
}


def deep_merge(base: dict, patch: dict) -> dict:
    out = copy.deepcopy(base)
    for k, v in (patch or {}).items():
        if isinstance(v, dict) and isinstance(out.get(k), dict):
            out[k] = deep_merge(out[k], v)
        else:
            out[k] = copy.deepcopy(v)
    return out


class _Section:
    def __init__(self, d: dict):
        object.__setattr__(self, "_d", d)

    def __getattr__(self, k):
        try:
            v = self._d[k]
        except KeyError as e:
            raise AttributeError(k) from e
        return _Section(v) if isinstance(v, dict) else v

    def __setattr__(self, k, v):
        self._d[k] = v

    def __getitem__(self, k):
        return self._d[k]

    def __setitem__(self, k, v):
        self._d[k] = v

    def get(self, k, default=None):
        return self._d.get(k, default)

    def to_dict(self):
        return copy.deepcopy(self._d)


class TrainConfig:
    def __init__(self, data: Optional[dict] = None):
        self.data = deep_merge(DEFAULTS, data or {})

    @classmethod
    def from_dict(cls, d):
        return cls(d)

    @classmethod
    def from_json(cls, path):
        with open(path) as f:
            return cls(json.load(f))

    @classmethod
    def from_yaml(cls, path):
        import yaml
        with open(path) as f:
            return cls(yaml.safe_load(f) or {})

    @classmethod
    def load(cls, path):
        return cls.from_json(path) if str(path).endswith(".json") else cls.from_yaml(path)

    def override(self, patch) -> "TrainConfig":
        """``patch``: dict, JSON text, or dotted ``a.b=value`` string."""
        if isinstance(patch, str):
            if patch.lstrip().startswith("{"):
                patch = json.loads(patch)
            else:
                key, _, val = patch.partition("=")
                try:
                    val = json.loads(val)
                except json.JSONDecodeError:
                    pass
                d = cur = {}
                parts = key.split(".")
                for p in parts[:-1]:
                    cur[p] = {}
                    cur = cur[p]
                cur[parts[-1]] = val
                patch = d
        self.data = deep_merge(self.data, patch)
        return self

    def __getattr__(self, k):
        if k in ("data",):
            raise AttributeError(k)
        if k in self.data:
            return _Section(self.data[k])
        raise AttributeError(k)

    def to_dict(self):
        return copy.deepcopy(self.data)

    def to_json(self, path=None):
        s = json.dumps(self.data, indent=2)
        if path:
            with open(path, "w") as f:
                f.write(s)
        return s

    def to_yaml(self, path=None):
        import yaml
        s = yaml.safe_dump(self.data, sort_keys=False)
        if path:
            with open(path, "w") as f:
                f.write(s)
        return s

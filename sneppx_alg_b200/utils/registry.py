"""Model registry with stages and lineage, prompt registry, evaluation monitor (the reference's ``mlflow_like.py``:
registry, lineage, prompt registry, AI gateway, eval monitor; C twin ``algorithms/model_zoo/registry.c:77-323`` with
versions / deprecation / search / save)."""
from __future__ import annotations

import json
import os
import time
from typing import Dict, List, Optional

STAGES = ("none", "staging", "production", "archived")


class ModelRegistry:
    def __init__(self, path: str):
        self.path = path
        self.data: Dict[str, dict] = json.load(open(path)) if os.path.exists(path) else {}

    def _flush(self):
        os.makedirs(os.path.dirname(os.path.abspath(self.path)), exist_ok=True)
        with open(self.path, "w") as f:
            json.dump(self.data, f, indent=1)

    def register(self, name: str, uri: str, metrics: dict = None, tags: List[str] = (), parent: Optional[str] = None,
                 run_id: Optional[str] = None) -> int:
        m = self.data.setdefault(name, {"versions": [], "created": time.time()})
        v = len(m["versions"]) + 1
        m["versions"].append({"version": v, "uri": uri, "metrics": metrics or {}, "tags": list(tags), "stage": "none",
                              "parent": parent, "run_id": run_id, "deprecated": False, "created": time.time()})
        self._flush()
        return v

    def get(self, name: str, version: Optional[int] = None, stage: Optional[str] = None) -> dict:
        vs = self.data[name]["versions"]
        if stage:
            vs = [v for v in vs if v["stage"] == stage]
        if version:
            vs = [v for v in vs if v["version"] == version]
        if not vs:
            raise KeyError(f"{name}: no version matches")
        return vs[-1]

    def transition(self, name: str, version: int, stage: str, archive_existing=True):
        assert stage in STAGES
        for v in self.data[name]["versions"]:
            if archive_existing and stage == "production" and v["stage"] == "production":
                v["stage"] = "archived"
        self.get(name, version)["stage"] = stage
        self._flush()

    def deprecate(self, name: str, version: int, reason: str = ""):
        v = self.get(name, version)
        v["deprecated"], v["deprecation_reason"] = True, reason
        self._flush()

    def search(self, query: str = "", tag: Optional[str] = None, min_metric: Optional[tuple] = None) -> List[dict]:
        out = []
        for name, m in self.data.items():
            for v in m["versions"]:
                if query.lower() in name.lower() and (tag is None or tag in v["tags"]) and \
                        (min_metric is None or v["metrics"].get(min_metric[0], float("-inf")) >= min_metric[1]):
                    out.append({"name": name, **v})
        return out

    def lineage(self, name: str, version: int) -> List[str]:
        """Chain of ancestors 'name:version' following ``parent`` links."""
        chain, cur = [], f"{name}:{version}"
        while cur:
            chain.append(cur)
            n, v = cur.rsplit(":", 1)
            cur = self.get(n, int(v)).get("parent")
        return chain


class PromptRegistry:
    def __init__(self):
        self.prompts: Dict[str, List[dict]] = {}

    def register(self, name: str, template: str, **meta) -> int:
        vs = self.prompts.setdefault(name, [])
        vs.append({"version": len(vs) + 1, "template": template, "meta": meta})
        return len(vs)

    def render(self, name: str, version: Optional[int] = None, **values) -> str:
        vs = self.prompts[name]
        return (vs[-1] if version is None else vs[version - 1])["template"].format(**values)


class EvalMonitor:
    """Tracks a metric stream and flags regressions against a trailing baseline."""

    def __init__(self, window=20, tolerance=0.05, higher_is_better=True):
        self.window, self.tol, self.hib, self.values = window, tolerance, higher_is_better, []

    def observe(self, v: float) -> bool:
        base = self.values[-self.window:]
        self.values.append(v)
        if len(base) < 3:
            return False
        mean = sum(base) / len(base)
        return (v < mean * (1 - self.tol)) if self.hib else (v > mean * (1 + self.tol))

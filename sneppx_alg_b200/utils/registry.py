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


class AIGateway:
    """Routes a request to one of several named providers (callables) with weighted selection, per-provider rate
    limits, fall-back to the next provider on failure and per-provider usage accounting (the reference's
    ``mlflow_like.py`` gateway: named routes in front of model endpoints)."""

    def __init__(self):
        self.routes = {}

    def add_route(self, route: str, provider: str, fn, weight: float = 1.0, rate_limit_per_s: float = 0.0):
        self.routes.setdefault(route, []).append({"provider": provider, "fn": fn, "weight": float(weight), "rate": rate_limit_per_s,
                                                  "tokens": rate_limit_per_s, "stamp": None, "calls": 0, "failures": 0})

    def _admit(self, p, now):
        if p["rate"] <= 0:
            return True
        if p["stamp"] is not None:
            p["tokens"] = min(p["rate"], p["tokens"] + (now - p["stamp"]) * p["rate"])
        p["stamp"] = now
        if p["tokens"] >= 1.0:
            p["tokens"] -= 1.0
            return True
        return False

    def query(self, route: str, payload, request_id: str = "", now: Optional[float] = None):
        """Providers are tried in an order fixed by the request id (weighted, so the same id maps to the same first
        choice); a provider that is over its rate or raises is skipped. Returns (provider name, result)."""
        import hashlib
        import time
        ps = self.routes.get(route)
        if not ps:
            raise KeyError(f"unknown route {route}")
        now = time.monotonic() if now is None else now
        h = int.from_bytes(hashlib.sha256(request_id.encode()).digest()[:8], "big") / 2 ** 64
        order, pool = [], list(ps)
        while pool:
            tot = sum(p["weight"] for p in pool)
            acc, pick = 0.0, pool[-1]
            for p in pool:
                acc += p["weight"] / tot
                if h < acc:
                    pick = p
                    break
            order.append(pick)
            pool.remove(pick)
        errors = []
        for p in order:
            if not self._admit(p, now):
                errors.append(f"{p['provider']}: rate limited")
                continue
            try:
                p["calls"] += 1
                return p["provider"], p["fn"](payload)
            except Exception as e:  # fall back to the next provider
                p["failures"] += 1
                errors.append(f"{p['provider']}: {e}")
        raise RuntimeError("all providers failed: " + "; ".join(errors))

    def usage(self, route: str):
        return {p["provider"]: {"calls": p["calls"], "failures": p["failures"]} for p in self.routes.get(route, [])}

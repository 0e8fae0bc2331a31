"""Model-serving control plane: versioned model registry with deploy / promote / rollback, weighted A/B traffic
split by request-id hash, dynamic batching queue (size / timeout), warm-up driven readiness, latency metrics with
p50 / p95 / p99 / rps and Prometheus text export, YAML hot reload. Mirrors the reference's ``ServingEngine`` and
``MetricsCollector`` (interface_bindings/serving_engine.py:49-815) and its C twin (net/http/serving_engine.c)."""
from __future__ import annotations

import hashlib
import os
import threading
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional


class MetricsCollector:
    def __init__(self, reservoir: int = 4096):
        self.lat = deque(maxlen=reservoir)
        self.ttft = deque(maxlen=reservoir)
        self.requests = 0
        self.errors = 0
        self.tokens_out = 0
        self.tokens_in = 0
        self.start = time.time()
        self._lock = threading.Lock()

    def record(self, latency_s: float, ok: bool = True, tokens_in: int = 0, tokens_out: int = 0,
               ttft_s: Optional[float] = None):
        with self._lock:
            self.requests += 1
            self.errors += 0 if ok else 1
            self.lat.append(latency_s)
            if ttft_s is not None:
                self.ttft.append(ttft_s)
            self.tokens_in += tokens_in
            self.tokens_out += tokens_out

    @staticmethod
    def _pct(values, q):
        if not values:
            return 0.0
        s = sorted(values)
        return s[min(len(s) - 1, int(q * (len(s) - 1) + 0.5))]

    def snapshot(self) -> Dict[str, float]:
        with self._lock:
            up = max(time.time() - self.start, 1e-9)
            return {"requests_total": self.requests, "errors_total": self.errors, "rps": self.requests / up,
                    "latency_p50": self._pct(self.lat, 0.5), "latency_p95": self._pct(self.lat, 0.95),
                    "latency_p99": self._pct(self.lat, 0.99), "ttft_p50": self._pct(self.ttft, 0.5),
                    "ttft_p99": self._pct(self.ttft, 0.99), "tokens_in_total": self.tokens_in,
                    "tokens_out_total": self.tokens_out, "output_tokens_per_s": self.tokens_out / up,
                    "uptime_s": up}

    def prometheus(self, prefix: str = "sneppx") -> str:
        lines = []
        for k, v in self.snapshot().items():
            kind = "counter" if k.endswith("_total") else "gauge"
            lines.append(f"# TYPE {prefix}_{k} {kind}")
            lines.append(f"{prefix}_{k} {v}")
        return "\n".join(lines) + "\n"


@dataclass
class ModelVersion:
    model_id: str
    version: str
    handler: Callable[..., Any]
    weight: float = 0.0
    status: str = "staged"          # staged | serving | retired
    created: float = field(default_factory=time.time)
    warm_ticks: int = 0


class ServingEngine:
    def __init__(self, warmup_ticks: int = 1, max_batch: int = 32, batch_timeout_ms: float = 2.0, config_path=None):
        self.models: Dict[str, Dict[str, ModelVersion]] = {}
        self.history: Dict[str, List[str]] = {}
        self.metrics = MetricsCollector()
        self.warmup_ticks, self.max_batch, self.batch_timeout_ms = warmup_ticks, max_batch, batch_timeout_ms
        self.config_path, self._mtime = config_path, 0.0
        self._lock = threading.Lock()
        self._queue: deque = deque()

    # ---- registry
    def register_model(self, model_id: str, version: str, handler, weight: float = 0.0) -> ModelVersion:
        mv = ModelVersion(model_id, version, handler, weight)
        with self._lock:
            self.models.setdefault(model_id, {})[version] = mv
        return mv

    def deploy(self, model_id: str, version: str, weight: float = 1.0) -> None:
        with self._lock:
            mv = self.models[model_id][version]
            mv.status, mv.weight = "serving", weight
            self.history.setdefault(model_id, []).append(version)

    def promote(self, model_id: str, version: str) -> None:
        """Give ``version`` all traffic."""
        with self._lock:
            for v, mv in self.models[model_id].items():
                if v == version:
                    mv.status, mv.weight = "serving", 1.0
                elif mv.status == "serving":
                    mv.status, mv.weight = "retired", 0.0
            self.history.setdefault(model_id, []).append(version)

    def rollback(self, model_id: str) -> Optional[str]:
        h = self.history.get(model_id, [])
        if len(h) < 2:
            return None
        h.pop()
        prev = h.pop()
        self.promote(model_id, prev)
        return prev

    def set_traffic(self, model_id: str, weights: Dict[str, float]) -> None:
        with self._lock:
            for v, w in weights.items():
                mv = self.models[model_id][v]
                mv.weight = w
                mv.status = "serving" if w > 0 else mv.status

    def list_models(self):
        return {m: {v: {"status": mv.status, "weight": mv.weight} for v, mv in vs.items()} for m, vs in self.models.items()}

    # ---- routing
    def route(self, model_id: str, request_id: str) -> ModelVersion:
        vs = [mv for mv in self.models[model_id].values() if mv.status == "serving" and mv.weight > 0]
        if not vs:
            raise KeyError(f"no serving version of '{model_id}'")
        tot = sum(mv.weight for mv in vs)
        h = int(hashlib.sha256(request_id.encode()).hexdigest()[:8], 16) / 0xFFFFFFFF * tot
        acc = 0.0
        for mv in sorted(vs, key=lambda m: m.version):
            acc += mv.weight
            if h <= acc:
                return mv
        return vs[-1]

    def infer(self, model_id: str, request_id: str, *args, **kw):
        t0 = time.perf_counter()
        ok = True
        try:
            mv = self.route(model_id, request_id)
            out = mv.handler(*args, **kw)
            mv.warm_ticks += 1
            return out
        except Exception:
            ok = False
            raise
        finally:
            self.metrics.record(time.perf_counter() - t0, ok)

    def ready(self) -> bool:
        serving = [mv for vs in self.models.values() for mv in vs.values() if mv.status == "serving"]
        return bool(serving) and all(mv.warm_ticks >= self.warmup_ticks for mv in serving)

    def warm_up(self, model_id: str, *args, **kw) -> None:
        for mv in self.models[model_id].values():
            if mv.status == "serving":
                for _ in range(self.warmup_ticks):
                    mv.handler(*args, **kw)
                    mv.warm_ticks += 1

    # ---- dynamic batching (size / timeout)
    def enqueue(self, item) -> None:
        self._queue.append((time.perf_counter(), item))

    def next_batch(self) -> List[Any]:
        if not self._queue:
            return []
        oldest = self._queue[0][0]
        if len(self._queue) >= self.max_batch or (time.perf_counter() - oldest) * 1e3 >= self.batch_timeout_ms:
            n = min(self.max_batch, len(self._queue))
            return [self._queue.popleft()[1] for _ in range(n)]
        return []

    # ---- YAML hot reload: flat dotted keys + "traffic:" block
    def maybe_reload(self) -> bool:
        if not self.config_path or not os.path.exists(self.config_path):
            return False
        m = os.path.getmtime(self.config_path)
        if m <= self._mtime:
            return False
        self._mtime = m
        import yaml
        with open(self.config_path) as f:
            cfg = yaml.safe_load(f) or {}
        self.max_batch = int(cfg.get("batch.max_size", cfg.get("max_batch", self.max_batch)))
        self.batch_timeout_ms = float(cfg.get("batch.timeout_ms", self.batch_timeout_ms))
        for model_id, weights in (cfg.get("traffic") or {}).items():
            if model_id in self.models:
                self.set_traffic(model_id, {str(k): float(v) for k, v in weights.items() if str(k) in self.models[model_id]})
        return True

"""Small classes behind reference names that need an object of their own kind.

Each class here answers to one public name of the reference's flat namespace with the constructor and methods that
name has there, on top of this package's own machinery. The flat namespace looks here before ``compat`` and
``compat_services``, which hold the rest.
"""
from __future__ import annotations

import collections
import json
import os
import threading
import time
import uuid
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .algorithms import npe as _npe
from .security import crypto as _crypto
from .security import services as _svc
from .security.model_watermark import BackdoorWatermark, WeightWatermark  # noqa: F401


# ------------------------------------------------------------------------------------------------ traffic limits
class SlidingWindowRateLimiter:
    """At most ``max_requests`` per key inside any ``window_seconds`` span, counted exactly from per-key timestamps
    (reference: interface_bindings/ddos_mitigation.py:103). The token bucket of ``security.services`` smooths
    bursts instead; this one forgets nothing inside the window."""

    def __init__(self, max_requests: int, window_seconds: float, clock: Callable[[], float] = time.monotonic):
        self.max_requests, self.window, self._clock = int(max_requests), float(window_seconds), clock
        self._seen: Dict[str, collections.deque] = {}
        self._lock = threading.Lock()

    def _trim(self, key: str, now: float) -> collections.deque:
        q = self._seen.setdefault(key, collections.deque())
        while q and now - q[0] >= self.window:
            q.popleft()
        return q

    def check(self, key: str) -> bool:
        """Counts the request and returns True when it is within the limit; a refused request is not counted."""
        with self._lock:
            q = self._trim(key, self._clock())
            if len(q) >= self.max_requests:
                return False
            q.append(self._clock())
            return True

    def get_count(self, key: str) -> int:
        with self._lock:
            return len(self._trim(key, self._clock()))


class SYNFloodDetector:
    """Flags a flood when more than ``threshold`` connection openings fall inside ``window`` seconds
    (reference: interface_bindings/ddos_mitigation.py:214)."""

    def __init__(self, threshold: int = 1000, window: float = 1.0, clock: Callable[[], float] = time.monotonic):
        self.threshold, self.window, self._clock = int(threshold), float(window), clock
        self._stamps: collections.deque = collections.deque()

    def _trim(self, now: float):
        while self._stamps and now - self._stamps[0] > self.window:
            self._stamps.popleft()

    def record_syn(self) -> bool:
        now = self._clock()
        self._stamps.append(now)
        self._trim(now)
        return len(self._stamps) > self.threshold

    def get_rate(self) -> float:
        self._trim(self._clock())
        return len(self._stamps) / self.window


# ------------------------------------------------------------------------------------------------ identities
class Authenticator:
    """Checks the ``Authorization`` header of a request (reference: interface_bindings/security_middleware.py:301).
    ``config`` has ``mode`` ("none", "bearer": a token listed in ``config.api_keys`` or equal to ``config.admin_key``;
    "api_key": a key that ``key_manager`` validates). ``authenticate`` returns a dict describing the caller, or None
    when the header does not pass."""

    def __init__(self, config=None, key_manager=None):
        if config is None:
            from .compat_services import AuthConfig
            config = AuthConfig()
        if config.mode not in ("none", "bearer", "api_key"):
            raise ValueError(f"unknown auth mode {config.mode!r}")
        self.config = config
        self.keys = key_manager if key_manager is not None or config.mode != "api_key" else ApiKeyManager()

    @property
    def enabled(self) -> bool:
        return self.config.mode != "none"

    @property
    def mode(self) -> str:
        return self.config.mode

    @staticmethod
    def _bearer(authorization: Optional[str]) -> Optional[str]:
        if not authorization:
            return None
        parts = authorization.strip().split(None, 1)
        if len(parts) == 2 and parts[0].lower() == "bearer" and parts[1].strip():
            return parts[1].strip()
        return None

    @staticmethod
    def _same(a: str, b: Optional[str]) -> bool:
        return bool(b) and _crypto.ct_equal(_crypto.sha256(a.encode()), _crypto.sha256(b.encode()))

    def authenticate(self, authorization: Optional[str]) -> Optional[Dict[str, Any]]:
        if not self.enabled:
            return {"mode": "none", "owner": "anonymous", "admin": False}
        token = self._bearer(authorization)
        if token is None:
            return None
        if self._same(token, getattr(self.config, "admin_key", None)):
            return {"mode": self.mode, "owner": "admin", "admin": True}
        if self.mode == "bearer":
            ok = False
            for k in getattr(self.config, "api_keys", ()):      # every entry is compared: no early exit on a match
                ok |= self._same(token, k)
            return {"mode": "bearer", "owner": "token", "admin": False} if ok else None
        info = self.keys.validate_key(token) if hasattr(self.keys, "validate_key") else (
            {"id": "key"} if self.keys.check(token) else None)
        return None if info is None else {"mode": "api_key", "owner": info.get("user_id") or info.get("name") or info["id"],
                                          "admin": False, "key": info}


from .security.network import IdentityManager  # noqa: E402,F401


# ------------------------------------------------------------------------------------------------ supply chain
@dataclass
class SBOMPart:
    name: str
    version: str
    supplier: Optional[str] = None
    licenses: List[str] = field(default_factory=list)
    hashes: Dict[str, str] = field(default_factory=dict)

    @property
    def purl(self) -> str:
        return f"pkg:pypi/{self.name.lower()}@{self.version}"


@dataclass
class SBOM:
    """Software bill of materials of one image or environment; ``to_cyclonedx_json`` gives the CycloneDX 1.4 document
    (reference: interface_bindings/container_security.py:66)."""

    name: str = "environment"
    version: str = "0"
    components: List[SBOMPart] = field(default_factory=list)
    serial: str = ""
    created: str = ""

    def __post_init__(self):
        self.serial = self.serial or f"urn:uuid:{uuid.uuid4()}"
        self.created = self.created or time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())

    @classmethod
    def from_packages(cls, packages: Dict[str, str], name: str = "environment") -> "SBOM":
        return cls(name=name, components=[SBOMPart(n, v) for n, v in sorted(packages.items())])

    def packages(self) -> Dict[str, str]:
        return {c.name: c.version for c in self.components}

    def to_cyclonedx_json(self) -> Dict[str, Any]:
        return {"bomFormat": "CycloneDX", "specVersion": "1.4", "serialNumber": self.serial, "version": 1,
                "metadata": {"timestamp": self.created, "component": {"type": "application", "name": self.name,
                                                                      "version": self.version}},
                "components": [{"type": "library", "name": c.name, "version": c.version, "purl": c.purl,
                                **({"supplier": {"name": c.supplier}} if c.supplier else {}),
                                **({"licenses": [{"license": {"id": l}} for l in c.licenses]} if c.licenses else {}),
                                **({"hashes": [{"alg": a, "content": h} for a, h in c.hashes.items()]} if c.hashes else {})}
                               for c in self.components]}


class CVEScanner:
    """Looks packages up in an advisory table (version ranges) with an on-disk result cache
    (reference: interface_bindings/container_security.py:122). The matching is ``security.pentest.VulnScanner``'s."""

    def __init__(self, cache_dir: Optional[str] = None, advisories=()):
        from .security.pentest import VulnScanner
        self._scanner = VulnScanner(advisories)
        self.cache_path = os.path.join(cache_dir, "cve_cache.json") if cache_dir else None
        self._cache: Dict[str, list] = {}
        if self.cache_path and os.path.exists(self.cache_path):
            with open(self.cache_path) as f:
                self._cache = json.load(f)

    def add_advisory(self, adv) -> None:
        self._scanner.add_advisory(adv)
        self._cache.clear()

    def scan_package(self, package: str, version: str) -> List[dict]:
        key = f"{package}=={version}"
        if key not in self._cache:
            self._cache[key] = self._scanner.scan({package: version})
            if self.cache_path:
                os.makedirs(os.path.dirname(self.cache_path), exist_ok=True)
                with open(self.cache_path, "w") as f:
                    json.dump(self._cache, f)
        return list(self._cache[key])

    def scan_sbom(self, sbom: SBOM) -> List[dict]:
        return [hit for c in sbom.components for hit in self.scan_package(c.name, c.version)]


class ContainerSecurity:
    """Per-image SBOM registry with recorded vulnerabilities and a compliance check against a policy
    ``{"max_severity": float, "max_count": int, "forbidden_packages": [...]}``
    (reference: interface_bindings/secure_updates.py:73)."""

    def __init__(self):
        self._sboms: Dict[str, dict] = {}
        self._vulns: Dict[str, List[dict]] = {}

    @staticmethod
    def generate_sbom(packages: List[Dict[str, str]]) -> dict:
        return SBOM.from_packages({p["name"]: p.get("version", "0") for p in packages}).to_cyclonedx_json()

    def register_sbom(self, image_id: str, sbom: dict) -> None:
        self._sboms[image_id] = sbom
        self._vulns.setdefault(image_id, [])

    def add_vulnerability(self, image_id: str, vuln: dict) -> None:
        self._vulns.setdefault(image_id, []).append(dict(vuln))

    def scan_cves(self, image_id: str) -> List[dict]:
        if image_id not in self._sboms:
            raise KeyError(f"no SBOM registered for {image_id}")
        present = {c["name"] for c in self._sboms[image_id].get("components", [])}
        return [v for v in self._vulns.get(image_id, []) if v.get("package") in present or "package" not in v]

    def is_compliant(self, image_id: str, policy: dict) -> bool:
        hits = self.scan_cves(image_id)
        present = {c["name"] for c in self._sboms[image_id].get("components", [])}
        if present & set(policy.get("forbidden_packages", ())):
            return False
        if len(hits) > policy.get("max_count", float("inf")):
            return False
        return all(float(v.get("severity", 0.0)) <= policy.get("max_severity", 10.0) for v in hits)


# ------------------------------------------------------------------------------------------------ attention state
class IncrementalAttentionState:
    """Online-softmax accumulator of one query per head: feed score / value chunks in any split and ``output`` equals
    softmax over all of them (reference: interface_bindings/paged_attention.py:350). Tensors: scores [H, k],
    values [H, k, D]."""

    def __init__(self, num_heads: int, head_dim: int, dtype=torch.float32, device=None):
        self.num_heads, self.head_dim = int(num_heads), int(head_dim)
        self.acc = torch.zeros(num_heads, head_dim, dtype=dtype, device=device)
        self.max = torch.full((num_heads, 1), float("-inf"), dtype=dtype, device=device)
        self.sum = torch.zeros(num_heads, 1, dtype=dtype, device=device)

    def update(self, scores: torch.Tensor, values: torch.Tensor) -> None:
        scores, values = scores.to(self.acc), values.to(self.acc)
        new_max = torch.maximum(self.max, scores.amax(-1, keepdim=True))
        keep = torch.exp(self.max - new_max)
        keep = torch.where(torch.isfinite(keep), keep, torch.zeros_like(keep))
        w = torch.exp(scores - new_max)
        self.acc = self.acc * keep + torch.einsum("hk,hkd->hd", w, values)
        self.sum = self.sum * keep + w.sum(-1, keepdim=True)
        self.max = new_max

    def logsumexp(self) -> torch.Tensor:
        return self.max + torch.log(self.sum)

    def output(self) -> torch.Tensor:
        return self.acc / torch.where(self.sum > 0, self.sum, torch.ones_like(self.sum))


# ------------------------------------------------------------------------------------------------ checkpoint record
@dataclass
class TensorRecord:
    """One tensor entry of a ``.sneppx`` checkpoint: shape, element type code, byte range in the file
    (reference: interface_bindings/checkpoint.py:27). ``TensorRecord.read_all(path)`` lists a file's records."""

    shape: tuple = ()
    ndim: int = 0
    dtype: int = 0
    data_offset: int = 0
    data_size: int = 0
    strides: tuple = ()

    def __post_init__(self):
        self.shape = tuple(int(d) for d in self.shape)
        self.ndim = self.ndim or len(self.shape)
        if not self.strides:
            s, acc = [], 1
            for d in reversed(self.shape):
                s.append(acc)
                acc *= d
            self.strides = tuple(reversed(s))

    @property
    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n

    @classmethod
    def read_all(cls, path: str) -> List["TensorRecord"]:
        from .checkpoint.sneppx_format import CheckpointReader
        out, offset = [], 0
        with CheckpointReader(path) as r:
            for i in range(r.num_tensors):
                shape, dtype, nbytes = r.tensor_info(i)
                out.append(cls(shape=shape, dtype=dtype, data_offset=offset, data_size=nbytes))
                offset += nbytes
        return out


# ------------------------------------------------------------------------------------------------ edge target
@dataclass
class EdgeDevice:
    """What the host CPU offers an edge deployment (reference: interface_bindings/edge_runtime.py:75)."""

    arch: str = ""
    cores: int = 1
    flags: frozenset = frozenset()
    memory_mb: int = 0

    @classmethod
    def detect(cls) -> "EdgeDevice":
        import platform
        flags: set = set()
        mem = 0
        try:
            for line in open("/proc/cpuinfo"):
                if line.startswith(("flags", "Features")):
                    flags = set(line.split(":", 1)[1].split())
                    break
            for line in open("/proc/meminfo"):
                if line.startswith("MemTotal"):
                    mem = int(line.split()[1]) // 1024
                    break
        except OSError:
            pass
        return cls(platform.machine(), os.cpu_count() or 1, frozenset(flags), mem)

    def supports_int8(self) -> bool:
        return bool(self.flags & {"avx2", "avx512_vnni", "avx_vnni", "asimddp", "neon", "asimd"})

    def supports_fp16(self) -> bool:
        return bool(self.flags & {"f16c", "avx512fp16", "fphp", "asimdhp"})

    def __repr__(self) -> str:
        return (f"EdgeDevice(arch={self.arch}, cores={self.cores}, int8={self.supports_int8()}, "
                f"fp16={self.supports_fp16()}, memory_mb={self.memory_mb})")


# ------------------------------------------------------------------------------------------------ experiment runs
@dataclass
class RunRecord:
    """What a tracker keeps of one run; a ``LocalBackend`` stores it as one JSON file."""

    run_id: str
    experiment: str = "default"
    name: str = ""
    params: Dict[str, Any] = field(default_factory=dict)
    metrics: Dict[str, List[Tuple[int, float]]] = field(default_factory=dict)
    tags: Dict[str, str] = field(default_factory=dict)
    artifacts: List[str] = field(default_factory=list)
    status: str = "running"
    started: float = 0.0
    ended: float = 0.0


class LocalBackend:
    """Directory of runs, one ``<run_id>.json`` each (reference: interface_bindings/experiment_tracker.py:66)."""

    def __init__(self, storage_dir: str = "experiments"):
        self.storage_dir = storage_dir
        os.makedirs(storage_dir, exist_ok=True)

    def _path(self, run_id: str) -> str:
        if os.sep in run_id or run_id.startswith("."):
            raise ValueError(f"bad run id {run_id!r}")
        return os.path.join(self.storage_dir, f"{run_id}.json")

    def save(self, run: RunRecord) -> None:
        tmp = self._path(run.run_id) + ".tmp"
        with open(tmp, "w") as f:
            json.dump(asdict(run), f, default=str)
        os.replace(tmp, self._path(run.run_id))

    def load(self, run_id: str) -> Optional[RunRecord]:
        try:
            with open(self._path(run_id)) as f:
                d = json.load(f)
        except FileNotFoundError:
            return None
        d["metrics"] = {k: [tuple(p) for p in v] for k, v in d.get("metrics", {}).items()}
        return RunRecord(**d)

    def list_runs(self, experiment_name: Optional[str] = None) -> List[RunRecord]:
        runs = [self.load(f[:-5]) for f in sorted(os.listdir(self.storage_dir)) if f.endswith(".json")]
        return [r for r in runs if r and (experiment_name is None or r.experiment == experiment_name)]

    def delete_run(self, run_id: str) -> None:
        try:
            os.remove(self._path(run_id))
        except FileNotFoundError:
            pass


class Tracker:
    """Tracker interface with the run kept in memory; nothing is written anywhere
    (reference: interface_bindings/experiment_tracker.py:110). Subclasses add a sink."""

    def __init__(self):
        self._run: Optional[RunRecord] = None

    @property
    def run(self) -> Optional[RunRecord]:
        return self._run

    def start_run(self, experiment_name: str = "default", run_name: str = "", params: Optional[dict] = None,
                  tags: Optional[dict] = None) -> RunRecord:
        self._run = RunRecord(uuid.uuid4().hex[:12], experiment_name, run_name, dict(params or {}), {}, dict(tags or {}),
                              [], "running", time.time())
        return self._run

    def log_metric(self, key: str, value: float, step: int = 0):
        self.log_metrics({key: value}, step)

    def log_metrics(self, metrics: Dict[str, float], step: int = 0):
        if self._run is not None:
            for k, v in metrics.items():
                self._run.metrics.setdefault(k, []).append((int(step), float(v)))

    def log_param(self, key: str, value: Any):
        self.log_params({key: value})

    def log_params(self, params: Dict[str, Any]):
        if self._run is not None:
            self._run.params.update(params)

    def log_artifact(self, path: str):
        if self._run is not None:
            self._run.artifacts.append(path)

    def set_tag(self, key: str, value: str):
        if self._run is not None:
            self._run.tags[key] = value

    def set_status(self, status: str):
        if self._run is not None:
            self._run.status = status

    def end_run(self):
        if self._run is not None:
            if self._run.status == "running":
                self._run.status = "finished"
            self._run.ended = time.time()


class LogTracker(Tracker):
    """Prints what it is told, one line per call (reference: interface_bindings/experiment_tracker.py:157)."""

    def __init__(self, stream=None):
        super().__init__()
        self._stream = stream

    def _say(self, text: str):
        print(text, file=self._stream, flush=True)

    def start_run(self, *a, **k):
        r = super().start_run(*a, **k)
        self._say(f"[run {r.run_id}] start experiment={r.experiment} name={r.name} params={r.params}")
        return r

    def log_metrics(self, metrics, step: int = 0):
        super().log_metrics(metrics, step)
        self._say(f"[step {step}] " + " ".join(f"{k}={float(v):.6g}" for k, v in metrics.items()))

    def end_run(self):
        super().end_run()
        if self._run is not None:
            self._say(f"[run {self._run.run_id}] {self._run.status} after {self._run.ended - self._run.started:.2f}s")


# ------------------------------------------------------------------------------------------------ data
class BatchCollator:
    """Pads 1-D samples to one length and stacks them; (input, target) pairs are collated side by side
    (reference: interface_bindings/data.py:84)."""

    def __init__(self, padding_value: int = 0, max_length: Optional[int] = None):
        self.padding_value, self.max_length = padding_value, max_length

    def _stack(self, items) -> torch.Tensor:
        ts = [torch.as_tensor(t) for t in items]
        if ts[0].dim() != 1:
            return torch.stack(ts)
        n = self.max_length or max(t.shape[0] for t in ts)
        out = ts[0].new_full((len(ts), n), self.padding_value)
        for i, t in enumerate(ts):
            m = min(n, t.shape[0])
            out[i, :m] = t[:m]
        return out

    def __call__(self, batch):
        if isinstance(batch[0], tuple):
            return tuple(self._stack([b[i] for b in batch]) for i in range(len(batch[0])))
        return self._stack(batch)


class WorkerPool:
    """``num_workers`` threads that take batches off a serving engine's dynamic-batching queue and hand them to
    ``run_batch`` (reference: interface_bindings/serving_engine.py:608). The queue is polled under one lock, so a
    batch goes to exactly one worker."""

    def __init__(self, engine, run_batch: Callable[[List[Any]], Any], num_workers: int = 2, poll_s: float = 0.001):
        self.engine, self.run_batch, self.num_workers, self.poll_s = engine, run_batch, int(num_workers), poll_s
        self._threads: List[threading.Thread] = []
        self._stop = threading.Event()
        self._take = threading.Lock()
        self.batches_done = 0
        self.errors: List[BaseException] = []

    def _loop(self):
        while not self._stop.is_set():
            with self._take:
                batch = self.engine.next_batch()
            if not batch:
                self._stop.wait(self.poll_s)
                continue
            try:
                self.run_batch(batch)
            except Exception as e:  # noqa: BLE001 - a failing batch must not end the worker
                self.errors.append(e)
            with self._take:
                self.batches_done += 1

    def start(self) -> None:
        if self._threads:
            return
        self._stop.clear()
        self._threads = [threading.Thread(target=self._loop, daemon=True, name=f"sx-worker-{i}") for i in range(self.num_workers)]
        for t in self._threads:
            t.start()

    def stop(self) -> None:
        self._stop.set()
        for t in self._threads:
            t.join(timeout=5.0)
        self._threads = []

    def __enter__(self):
        self.start()
        return self

    def __exit__(self, *exc):
        self.stop()


# ------------------------------------------------------------------------------------------------ compute DAGs
_ELEMENTWISE = {"add": torch.add, "sub": torch.sub, "mul": torch.mul, "div": torch.div, "relu": torch.relu,
                "gelu": torch.nn.functional.gelu, "silu": torch.nn.functional.silu, "tanh": torch.tanh,
                "sigmoid": torch.sigmoid, "exp": torch.exp, "neg": torch.neg, "clip": None}


class GraphNode:
    """Node of a compute DAG built with Python operators (reference: interface_bindings/graph_compiler.py:75).
    ``evaluate(feeds)`` runs the DAG with each node computed once; ``elementwise_clusters(root)`` groups chains of
    element-wise nodes into ``FusedNode`` s."""

    _count = 0

    def __init__(self, op: str, inputs: Sequence["GraphNode"] = (), value: Any = None, name: Optional[str] = None,
                 attrs: Optional[dict] = None):
        GraphNode._count += 1
        self.op, self.inputs, self.value, self.attrs = op, tuple(inputs), value, dict(attrs or {})
        self.name = name or f"{op}_{GraphNode._count}"

    @staticmethod
    def input_(name: str = "input") -> "GraphNode":
        return GraphNode("input", name=name)

    @staticmethod
    def constant(value: Any, name: Optional[str] = None) -> "GraphNode":
        return GraphNode("constant", value=torch.as_tensor(value), name=name)

    @staticmethod
    def parameter(value: Any, name: Optional[str] = None) -> "GraphNode":
        return GraphNode("parameter", value=torch.as_tensor(value), name=name)

    @staticmethod
    def clip(x: "GraphNode", lo: float, hi: float) -> "GraphNode":
        return GraphNode("clip", (x,), attrs={"lo": lo, "hi": hi})

    @staticmethod
    def _lift(x) -> "GraphNode":
        return x if isinstance(x, GraphNode) else GraphNode.constant(x)

    def __add__(self, other):
        return GraphNode("add", (self, self._lift(other)))

    def __sub__(self, other):
        return GraphNode("sub", (self, self._lift(other)))

    def __mul__(self, other):
        return GraphNode("mul", (self, self._lift(other)))

    def __truediv__(self, other):
        return GraphNode("div", (self, self._lift(other)))

    def __matmul__(self, other):
        return GraphNode("matmul", (self, self._lift(other)))

    def __neg__(self):
        return GraphNode("neg", (self,))

    def apply(self, op: str) -> "GraphNode":
        if op not in _ELEMENTWISE or op == "clip":
            raise ValueError(f"unknown unary op {op!r}")
        return GraphNode(op, (self,))

    relu = lambda self: self.apply("relu")        # noqa: E731
    gelu = lambda self: self.apply("gelu")        # noqa: E731
    tanh = lambda self: self.apply("tanh")        # noqa: E731
    sigmoid = lambda self: self.apply("sigmoid")  # noqa: E731

    @property
    def is_elementwise(self) -> bool:
        return self.op in _ELEMENTWISE

    def toposort(self) -> List["GraphNode"]:
        order, seen, stack = [], set(), [(self, False)]
        while stack:
            n, done = stack.pop()
            if done:
                order.append(n)
            elif id(n) not in seen:
                seen.add(id(n))
                stack.append((n, True))
                stack.extend((i, False) for i in reversed(n.inputs))
        return order

    def compute(self, args: Sequence[torch.Tensor]) -> torch.Tensor:
        if self.op == "matmul":
            return args[0] @ args[1]
        if self.op == "clip":
            return args[0].clamp(self.attrs["lo"], self.attrs["hi"])
        return _ELEMENTWISE[self.op](*args)

    def evaluate(self, feeds: Optional[Dict[str, torch.Tensor]] = None) -> torch.Tensor:
        feeds, vals = feeds or {}, {}
        for n in self.toposort():
            if n.op == "input":
                vals[id(n)] = feeds[n.name]
            elif n.op in ("constant", "parameter"):
                vals[id(n)] = feeds.get(n.name, n.value)
            else:
                vals[id(n)] = n.compute([vals[id(i)] for i in n.inputs])
        return vals[id(self)]

    def __repr__(self) -> str:
        return f"GraphNode({self.name}: {self.op}({', '.join(i.name for i in self.inputs)}))"


class FusedNode:
    """A chain of element-wise nodes run as one step: the members in order, each fed by the previous one or by
    nodes outside the cluster (reference: interface_bindings/graph_compiler.py:215)."""

    def __init__(self, members: List[GraphNode], name: str = "fused"):
        if not members or not all(m.is_elementwise for m in members):
            raise ValueError("a fused node is a non-empty list of element-wise nodes")
        self.members, self.name = list(members), name
        inside = {id(m) for m in self.members}
        self.external_inputs = [i for m in self.members for i in m.inputs if id(i) not in inside]
        self.output = self.members[-1]

    def run(self, external: Dict[int, torch.Tensor]) -> torch.Tensor:
        """``external`` maps id(node) of every outside input to its value."""
        vals = dict(external)
        for m in self.members:
            vals[id(m)] = m.compute([vals[id(i)] for i in m.inputs])
        return vals[id(self.output)]

    def __repr__(self) -> str:
        return f"FusedNode({self.name}: {'+'.join(m.op for m in self.members)})"


def elementwise_clusters(root: GraphNode) -> List[FusedNode]:
    """Maximal single-consumer chains of element-wise nodes under ``root`` (two or more members each)."""
    order = root.toposort()
    users: Dict[int, int] = collections.Counter(id(i) for n in order for i in n.inputs)
    clusters, taken = [], set()
    for n in reversed(order):
        if id(n) in taken or not n.is_elementwise:
            continue
        chain = [n]
        while True:
            nxt = [i for i in chain[0].inputs if i.is_elementwise and users[id(i)] == 1 and id(i) not in taken]
            if len(nxt) != 1:
                break
            chain.insert(0, nxt[0])
        if len(chain) > 1:
            taken.update(id(c) for c in chain)
            clusters.append(FusedNode(chain, name=f"fused_{len(clusters)}"))
    return clusters


class TensorExpr:
    """Tensor expression tree with named constructors (reference: interface_bindings/c_tensor_expr.py:16)."""

    def __init__(self, op: str, *inputs: "TensorExpr", value: Optional[torch.Tensor] = None, name: str = ""):
        self.op, self.inputs, self.value, self.name = op, inputs, value, name

    @staticmethod
    def constant(data) -> "TensorExpr":
        return TensorExpr("const", value=torch.as_tensor(data))

    @staticmethod
    def parameter(data, name: str = "") -> "TensorExpr":
        return TensorExpr("param", value=torch.as_tensor(data), name=name)

    @staticmethod
    def add(a, b) -> "TensorExpr":
        return TensorExpr("add", a, b)

    @staticmethod
    def mul(a, b) -> "TensorExpr":
        return TensorExpr("mul", a, b)

    @staticmethod
    def matmul(a, b) -> "TensorExpr":
        return TensorExpr("matmul", a, b)

    @staticmethod
    def relu(x) -> "TensorExpr":
        return TensorExpr("relu", x)

    def evaluate(self, bindings: Optional[dict] = None) -> torch.Tensor:
        plan = TensorExprCompiler().compile(self)
        return TensorExprCompiler.run(plan, bindings)

    def __repr__(self) -> str:
        return f"TensorExpr({self.op}" + (f", {len(self.inputs)} inputs)" if self.inputs else ")")


class TensorExprCompiler:
    """Flattens an expression tree into a plan: a list of ``(op, input slots, payload)`` in execution order, with
    shared sub-trees planned once; ``run(plan, bindings)`` executes it (bindings override named parameters)."""

    _FN = {"add": torch.add, "mul": torch.mul, "matmul": torch.matmul, "relu": torch.relu}

    def __init__(self):
        self.plan: List[tuple] = []

    def compile(self, expr: TensorExpr) -> List[tuple]:
        self.plan, slot = [], {}

        def visit(node: TensorExpr) -> int:
            if id(node) in slot:
                return slot[id(node)]
            ins = tuple(visit(i) for i in node.inputs)
            payload = (node.name, node.value) if node.op in ("const", "param") else None
            self.plan.append((node.op, ins, payload))
            slot[id(node)] = len(self.plan) - 1
            return slot[id(node)]

        visit(expr)
        return self.plan

    @classmethod
    def run(cls, plan: List[tuple], bindings: Optional[dict] = None) -> torch.Tensor:
        bindings, vals = bindings or {}, []
        for op, ins, payload in plan:
            if payload is not None:
                name, value = payload
                vals.append(torch.as_tensor(bindings[name]) if name and name in bindings else value)
            else:
                vals.append(cls._FN[op](*(vals[i] for i in ins)))
        return vals[-1]


# ------------------------------------------------------------------------------------------------ device handles
class DeviceContext:
    """``with DeviceContext(i):`` makes device ``i`` current and restores the previous one on exit
    (reference: interface_bindings/cuda_device.py:118)."""

    def __init__(self, device_id: int):
        self.device_id, self._prev = int(device_id), None

    def __enter__(self):
        if torch.cuda.is_available():
            self._prev = torch.cuda.current_device()
            torch.cuda.set_device(self.device_id)
        return self

    def __exit__(self, *exc):
        if self._prev is not None:
            torch.cuda.set_device(self._prev)
            self._prev = None


class CUDADriver:
    """Handle-style access to devices, streams, events and raw device memory
    (reference: interface_bindings/driver_bindings.py:36). Handles are small dicts that own the torch object; a call
    on a host without a GPU returns None (creation) or -1 (status), never raises."""

    def __init__(self):
        self._allocations: Dict[int, torch.Tensor] = {}

    @staticmethod
    def is_available() -> bool:
        return torch.cuda.is_available()

    def get_device_count(self) -> int:
        return torch.cuda.device_count() if self.is_available() else 0

    def get_device_props(self, dev_id: int = 0):
        from . import device as _device
        return _device.properties(dev_id)

    def set_device(self, dev_id: int) -> int:
        if not self.is_available() or not 0 <= dev_id < torch.cuda.device_count():
            return -1
        torch.cuda.set_device(dev_id)
        return 0

    def get_device(self) -> int:
        return torch.cuda.current_device() if self.is_available() else -1

    def create_context(self, device_id: int = 0) -> Optional[dict]:
        if self.set_device(device_id) != 0:
            return None
        torch.cuda.init()
        return {"device": device_id, "error": 0}

    def destroy_context(self, ctx: dict):
        ctx["device"] = -1

    def context_error(self, ctx: dict) -> int:
        return int(ctx.get("error", 0))

    def stream_create(self, priority: int = 0) -> Optional[dict]:
        return {"stream": torch.cuda.Stream(priority=priority)} if self.is_available() else None

    def stream_destroy(self, stream: dict):
        stream.pop("stream", None)

    def stream_synchronize(self, stream: dict) -> int:
        if "stream" not in stream:
            return -1
        stream["stream"].synchronize()
        return 0

    def event_create(self) -> Optional[dict]:
        return {"event": torch.cuda.Event(enable_timing=True)} if self.is_available() else None

    def event_destroy(self, event: dict):
        event.pop("event", None)

    def event_record(self, event: dict, stream: Optional[dict] = None) -> int:
        if "event" not in event:
            return -1
        event["event"].record(stream["stream"] if stream else None)
        return 0

    def event_synchronize(self, event: dict) -> int:
        if "event" not in event:
            return -1
        event["event"].synchronize()
        return 0

    def event_elapsed_ms(self, start: dict, end: dict) -> float:
        return float(start["event"].elapsed_time(end["event"]))

    def mem_alloc(self, nbytes: int) -> Optional[int]:
        if not self.is_available() or nbytes <= 0:
            return None
        t = torch.empty(int(nbytes), dtype=torch.uint8, device="cuda")
        self._allocations[t.data_ptr()] = t
        return t.data_ptr()

    def mem_free(self, dev_ptr: int):
        self._allocations.pop(dev_ptr, None)


# ------------------------------------------------------------------------------------------------ NPE front end
class NPECompiler:
    """Compiles a list of named operations ``{"type": "matmul", "args": ["x", "w1"], "dest": "h"}`` into a register
    program for the NPE virtual machine (reference: interface_bindings/algo_npe.py:45). ``"x"`` (or ``"input"``) is
    the VM's input register; every other name that is used before it is defined must be in ``weights`` and is laid
    out in program memory and brought in with LOAD. Registers are reused once their value has no later use."""

    OPCODES = {"add": _npe.Op.ADD, "sub": _npe.Op.SUB, "mul": _npe.Op.MUL, "div": _npe.Op.DIV, "matmul": _npe.Op.MATMUL,
               "relu": _npe.Op.RELU, "gelu": _npe.Op.GELU, "silu": _npe.Op.SILU, "tanh": _npe.Op.TANH,
               "sigmoid": _npe.Op.SIGMOID, "softmax": _npe.Op.SOFTMAX, "layernorm": _npe.Op.LAYERNORM,
               "neg": _npe.Op.NEG, "exp": _npe.Op.EXP, "nop": _npe.Op.NOP}
    INPUT_NAMES = ("x", "input")

    def compile(self, operations: List[dict], weights: Optional[Dict[str, torch.Tensor]] = None, output: Optional[str] = None,
                device=None) -> _npe.Program:
        weights = weights or {}
        ops = [o for o in operations if o.get("type", "nop") != "nop"]
        for o in ops:
            if o["type"] not in self.OPCODES:
                raise ValueError(f"unknown operation type {o['type']!r}")
        output = output or (ops[-1]["dest"] if ops else None)
        last_use: Dict[str, int] = {}
        for i, o in enumerate(ops):
            for a in o.get("args", []):
                last_use[a] = i
        if output is not None:
            last_use[output] = len(ops)
        needed = [n for n in dict.fromkeys(a for o in ops for a in o.get("args", []))
                  if n not in self.INPUT_NAMES and n not in {p["dest"] for p in ops}]
        missing = [n for n in needed if n not in weights]
        if missing:
            raise KeyError(f"operands without a value: {missing}")
        offsets, total = {}, 0
        for n in needed:
            offsets[n] = total
            total += weights[n].numel()
        prog = _npe.Program(total + 1, max(32, 2 * len(ops) + len(needed) + 2), device=device)
        with torch.no_grad():
            for n in needed:
                prog.memory[offsets[n]: offsets[n] + weights[n].numel()] = weights[n].reshape(-1).to(prog.memory)
        reg: Dict[str, int] = {n: 0 for n in self.INPUT_NAMES}
        free = collections.deque(range(1, _npe.NUM_REGS))     # oldest-freed first, so a register is reused as late as possible

        def take(name: str) -> int:
            if not free:
                raise OverflowError("more than 15 values are live at once")
            reg[name] = free.popleft()
            return reg[name]

        def release(step: int, names):
            for n in set(names):
                if n not in self.INPUT_NAMES and last_use.get(n, -1) <= step and n in reg:
                    free.append(reg.pop(n))

        I = _npe.Instruction  # noqa: E741

        def load(a: str):
            w = weights[a]
            shape = (w.shape[0], w.shape[1]) if w.dim() == 2 else (w.numel(), 0)
            prog.append(I(_npe.Op.LOAD, take(a), immediate=offsets[a], shape_a=shape))

        for a in needed:                       # constants go in up front while half the registers stay free, so that
            if len(free) > _npe.NUM_REGS // 2:  # MATMUL / ADD / activation chains stay adjacent for the fusion pass
                load(a)
        for step, o in enumerate(ops):
            args = o.get("args", [])
            for a in args:
                if a not in reg:
                    load(a)
            srcs = [reg[a] for a in args] + [0, 0]
            release(step, args)
            prog.append(I(self.OPCODES[o["type"]], take(o["dest"]), srcs[0], srcs[1]))
            if last_use.get(o["dest"], -1) <= step and o["dest"] != output:
                release(step, [o["dest"]])
        if output is not None:
            prog.append(I(_npe.Op.STORE, a=reg[output], immediate=total))
        prog.append(I(_npe.Op.HALT))
        return prog

    def jit_optimize(self, program: _npe.Program, profile: Optional[_npe.JITProfile] = None) -> _npe.Program:
        """Dead-code elimination, MATMUL+ADD(+activation) fusion and, with a profile, hot-path specialisation."""
        return _npe.jit_optimize(profile, program)


class NPEVerify:
    """Static checks of an NPE program (reference: interface_bindings/algo_npe.py:129)."""

    def verify(self, program: _npe.Program) -> Tuple[bool, List[str]]:
        return _npe.verify_program(program)

    def check_bounds(self, program: _npe.Program, max_ops: int = 1000) -> bool:
        return len(program.instructions) <= max_ops

    def check_types(self, program: _npe.Program, var_types: Optional[Dict[int, str]] = None) -> List[str]:
        """Registers read before anything wrote them (register 0 holds the input). ``var_types`` may name further
        registers that are defined on entry."""
        written, errors = {0} | set(var_types or ()), []
        reads = {_npe.Op.STORE: ("a",), _npe.Op.MATMUL: ("a", "b"), _npe.Op.ATTENTION: ("a", "b", "immediate"),
                 _npe.Op.FUSED_LINEAR: ("a", "b")}
        for i, ins in enumerate(program.instructions):
            op = ins.opcode
            if op in (_npe.Op.NOP, _npe.Op.HALT, _npe.Op.LOAD):
                fields: tuple = ()
            elif op in reads:
                fields = reads[op]
            elif op in _npe._BINARY or op in (_npe.Op.MSE, _npe.Op.CROSSENTROPY, _npe.Op.CONCAT):
                fields = ("a", "b")
            else:
                fields = ("a",)
            for f in fields:
                r = getattr(ins, f)
                if r not in written:
                    errors.append(f"Instr {i}: register {r} read before it is written")
            if op not in (_npe.Op.STORE, _npe.Op.HALT, _npe.Op.NOP, _npe.Op.BRANCH):
                written.add(ins.dest)
        return errors


# ------------------------------------------------------------------------------------------------ accessors
_profiler_lock = threading.Lock()
_profiler = None


def get_profiler():
    """The process-wide profiler (reference: interface_bindings/profiler.py:90)."""
    global _profiler
    with _profiler_lock:
        if _profiler is None:
            from .utils.observability import Profiler
            _profiler = Profiler()
        return _profiler


def create_vizmon(history: int = 1024):
    """A monitor with its server not started (reference: interface_bindings/vizmon.py:314)."""
    from .utils.vizmon import VizMon
    return VizMon(history)


def start_dashboard(port: int = 8300, host: str = "127.0.0.1"):
    """A monitor with its HTTP / WebSocket server running on ``port``; ``.stop()`` shuts it down
    (reference: interface_bindings/vizmon.py:304)."""
    vm = create_vizmon()
    vm.serve(host=host, port=port)
    return vm


_launcher = None


def get_launcher():
    """The process-wide kernel launcher table (reference: interface_bindings/cuda_kernels.py:151)."""
    global _launcher
    if _launcher is None:
        from .compat_services import KernelLauncher
        _launcher = KernelLauncher()
    return _launcher


# ------------------------------------------------------------------------------------------------ algorithm fronts
class ARCFForward:
    """Bounded forward propagation of the ARC family: every layer is ``clip(x W^T + b)`` with the output clamped to
    ``[-bound, bound]``, so a perturbation of the input can move an activation by at most ``2 * bound``
    (reference: interface_bindings/algo_arc.py:38). Weights are [out, in]."""

    bound = 10.0

    @classmethod
    def forward(cls, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        return torch.nn.functional.linear(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype)).clamp(-cls.bound, cls.bound)

    @classmethod
    def forward_layers(cls, x: torch.Tensor, layers: Sequence) -> torch.Tensor:
        """``layers``: (weight, bias) pairs or bare weights; ReLU between layers, none after the last."""
        for i, layer in enumerate(layers):
            w, b = layer if isinstance(layer, (tuple, list)) else (layer, None)
            x = cls.forward(x, w, b)
            if i + 1 < len(layers):
                x = torch.relu(x)
        return x


class ARCAdversarialTrainGraph:
    """The two forward paths of adversarial training over one weight list: the clean input and the input moved by
    ``attack_epsilon`` along the sign of the gradient of the clean output's squared norm
    (reference: interface_bindings/algo_arc.py:111). ``build`` returns (clean output, adversarial output)."""

    def __init__(self, attack_epsilon: float = 0.01):
        self.attack_epsilon = float(attack_epsilon)

    def build(self, weights: List[torch.Tensor], x_clean: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        x = x_clean.detach().clone().requires_grad_(True)
        clean = ARCFForward.forward_layers(x, weights)
        (g,) = torch.autograd.grad(clean.float().pow(2).sum(), x)
        x_adv = (x_clean + self.attack_epsilon * g.sign()).detach()
        return ARCFForward.forward_layers(x_clean, weights), ARCFForward.forward_layers(x_adv, weights)


class FMSync:
    """Reductions over a list of per-node tensors held by one process, and over the process group when one is
    initialised (reference: interface_bindings/algo_fm.py:83)."""

    OPS = {"sum": torch.distributed.ReduceOp.SUM, "max": torch.distributed.ReduceOp.MAX, "min": torch.distributed.ReduceOp.MIN}

    @classmethod
    def all_reduce(cls, tensor: torch.Tensor, op: str = "sum") -> torch.Tensor:
        if op not in cls.OPS and op != "mean":
            raise ValueError(f"unknown reduction {op!r}")
        import torch.distributed as dist
        out = tensor.clone()
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(out, cls.OPS["sum" if op == "mean" else op])
            if op == "mean":
                out /= dist.get_world_size()
        return out

    @staticmethod
    def federated_avg(local_tensors: List[torch.Tensor], weights: Optional[Sequence[float]] = None) -> torch.Tensor:
        from .algorithms.fm import federated_average
        return federated_average(list(local_tensors), weights)


class SERExpert(torch.nn.Module):
    """One expert of a mixture layer: ``gelu(x W1 + b1) W2 + b2`` back to the input width
    (reference: interface_bindings/algo_ser.py:15)."""

    def __init__(self, expert_id: int, input_dim: int, hidden_dim: int, dtype=None, device=None):
        super().__init__()
        self.expert_id = int(expert_id)
        self.up = torch.nn.Linear(input_dim, hidden_dim, dtype=dtype, device=device)
        self.down = torch.nn.Linear(hidden_dim, input_dim, dtype=dtype, device=device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down(torch.nn.functional.gelu(self.up(x)))


# ------------------------------------------------------------------------------------------------ small records
class CUDADeviceProps:
    """Properties of one CUDA device; ``CUDADeviceProps.query(i)`` fills them from the driver
    (reference: interface_bindings/driver_bindings.py:16)."""

    def __init__(self, name: str = "", global_mem: int = 0, shared_mem: int = 0, warp_size: int = 32, max_threads: int = 1024,
                 sm_count: int = 0, compute_major: int = 0, compute_minor: int = 0, has_tensor_cores: bool = False):
        self.name, self.global_mem, self.shared_mem, self.warp_size = name, global_mem, shared_mem, warp_size
        self.max_threads, self.sm_count = max_threads, sm_count
        self.compute_major, self.compute_minor, self.has_tensor_cores = compute_major, compute_minor, has_tensor_cores

    @classmethod
    def query(cls, index: int = 0) -> "CUDADeviceProps":
        p = torch.cuda.get_device_properties(index)
        return cls(p.name, p.total_memory, getattr(p, "shared_memory_per_block_optin", 0), p.warp_size,
                   p.max_threads_per_multi_processor, p.multi_processor_count, p.major, p.minor, p.major >= 7)

    def __repr__(self) -> str:
        return (f"CUDADeviceProps({self.name!r}, sm_{self.compute_major}{self.compute_minor}, {self.sm_count} SMs, "
                f"{self.global_mem >> 20} MiB)")


@dataclass
class DeviceInfo:
    """One entry of a hardware probe: a device kind, whether it can be used here and why
    (reference: interface_bindings/hw_backends.py:65)."""

    name: str
    available: bool
    kind: str = "cpu"
    detail: str = ""
    priority: int = 0

    @classmethod
    def probe(cls) -> List["DeviceInfo"]:
        out = [cls("cpu", True, "cpu", f"{os.cpu_count()} cores", 0)]
        if torch.cuda.is_available():
            for i in range(torch.cuda.device_count()):
                p = torch.cuda.get_device_properties(i)
                out.append(cls(p.name, True, "cuda", f"sm_{p.major}{p.minor}, {p.total_memory >> 30} GiB", 10))
        else:
            out.append(cls("cuda", False, "cuda", "no CUDA device visible", 10))
        return sorted(out, key=lambda d: -d.priority)


class GemmConfig:
    """Tile shape of a matrix product (reference: interface_bindings/c_simd_gemm.py:82). ``create_gemm`` returns a
    callable product ``(a, b) -> a @ b``; on CUDA bf16 operands it is this package's tensor-core GEMM, whose tile
    shape is fixed by the kernel, elsewhere a blocked product with these tiles."""

    def __init__(self, tile_m: int = 64, tile_n: int = 64, tile_k: int = 64, use_strassen: bool = False,
                 strassen_threshold: int = 128):
        self.tile_m, self.tile_n, self.tile_k = tile_m, tile_n, tile_k
        self.use_strassen, self.strassen_threshold = use_strassen, strassen_threshold

    def create_gemm(self) -> Callable[[torch.Tensor, torch.Tensor], torch.Tensor]:
        def product(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
            if a.is_cuda and a.dtype == torch.bfloat16:
                from .ops.gemm import gemm
                return gemm(a, b.t().contiguous())
            out = torch.zeros(a.shape[0], b.shape[1], dtype=torch.float32, device=a.device)
            for k0 in range(0, a.shape[1], self.tile_k):
                for m0 in range(0, a.shape[0], self.tile_m):
                    for n0 in range(0, b.shape[1], self.tile_n):
                        out[m0:m0 + self.tile_m, n0:n0 + self.tile_n] += (
                            a[m0:m0 + self.tile_m, k0:k0 + self.tile_k].float() @ b[k0:k0 + self.tile_k, n0:n0 + self.tile_n].float())
            return out.to(a.dtype)
        return product


class ConstantTimeOps:
    """Selections and table reads whose memory access pattern and branch pattern do not depend on the secret
    (reference: interface_bindings/crypto_asm.py:203). Integers are treated as 64-bit words."""

    MASK = (1 << 64) - 1

    @classmethod
    def ct_select(cls, a: int, b: int, cond: bool) -> int:
        m = -int(bool(cond)) & cls.MASK
        return (a & m) | (b & ~m & cls.MASK)

    @classmethod
    def ct_swap(cls, a: int, b: int, cond: bool) -> Tuple[int, int]:
        t = (-int(bool(cond)) & cls.MASK) & (a ^ b)
        return a ^ t, b ^ t

    @staticmethod
    def cache_const_lookup(table: bytes, index: int) -> int:
        """Reads every entry and keeps the one at ``index``."""
        if not 0 <= index < len(table):
            raise IndexError(index)
        out = 0
        for i, v in enumerate(table):
            diff = i ^ index
            is_eq = ((diff | -diff) >> 63) + 1          # 1 when diff == 0, else 0, without a comparison
            out |= v & -is_eq & 0xFF
        return out


# ------------------------------------------------------------------------------------------------ ONNX records
from .onnx import toolkit as _onnx  # noqa: E402


def _onnx_dtype(dtype) -> int:
    import numpy as np
    return dtype if isinstance(dtype, int) else _onnx._DT[np.dtype(dtype)]


class OnnxTensor(_onnx.ValueInfo):
    """Name, element type and shape of a graph input / output / intermediate: a ``ValueInfoProto``
    (reference: interface_bindings/onnx_export.py:233). ``dtype`` is a NumPy type name or an ONNX type code."""

    def __init__(self, name: str, dtype="float32", shape: Sequence = (), doc_string: str = ""):
        super().__init__(name, _onnx_dtype(dtype), tuple(shape))
        self.doc_string = doc_string

    def to_dict(self) -> Dict[str, Any]:
        return {"name": self.name, "elem_type": self.dtype, "shape": list(self.shape), "doc_string": self.doc_string}

    def to_proto(self) -> bytes:
        return self.serialize()


class OnnxInitializer(_onnx.Tensor):
    """A constant tensor of the graph with its bytes: a ``TensorProto``
    (reference: interface_bindings/onnx_export.py:265)."""

    def __init__(self, name: str, data, dtype=None):
        import numpy as np
        arr = np.asarray(data.detach().cpu().numpy() if isinstance(data, torch.Tensor) else data)
        super().__init__(name, arr.astype(dtype) if dtype is not None else arr)

    def to_dict(self) -> Dict[str, Any]:
        return {"name": self.name, "dims": list(self.data.shape), "data_type": _onnx._DT[self.data.dtype],
                "nbytes": int(self.data.nbytes)}

    def to_proto(self) -> bytes:
        return self.serialize()


# ------------------------------------------------------------------------------------------------ runs, streams, keys
class Run:
    """One training run as an object: ``with Run("exp", params=...) as r: r.log_metric("loss", x, step)``
    (reference: interface_bindings/experiment.py:45). Every mutator returns the run, so calls chain; ``to_dict`` /
    ``save(dir)`` / ``Run.load(path)`` round-trip it as JSON."""

    def __init__(self, experiment_name: str = "default", run_id: Optional[str] = None, params: Optional[Dict[str, Any]] = None):
        self.experiment_name, self.run_id = experiment_name, run_id or uuid.uuid4().hex[:12]
        self.params: Dict[str, Any] = dict(params or {})
        self.metrics: List[Dict[str, Any]] = []
        self.artifacts: List[str] = []
        self.tags: List[str] = []
        self.status, self.started_at, self.ended_at, self.error = "created", None, None, None

    @staticmethod
    def _now() -> str:
        return time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())

    def __enter__(self) -> "Run":
        return self.start()

    def __exit__(self, exc_type, exc, tb) -> bool:
        if exc is not None:
            self.fail(repr(exc))
        else:
            self.finish()
        return False

    def start(self) -> "Run":
        self.status, self.started_at = "running", self.started_at or self._now()
        return self

    def finish(self) -> "Run":
        if self.status != "failed":
            self.status = "finished"
        self.ended_at = self._now()
        return self

    def fail(self, error: str) -> "Run":
        self.status, self.error, self.ended_at = "failed", error, self._now()
        return self

    def log_params(self, params: Dict[str, Any]) -> "Run":
        self.params.update(params)
        return self

    def log_metric(self, key: str, value: Any, step: Optional[int] = None) -> "Run":
        self.metrics.append({"key": key, "value": float(value), "step": step, "time": time.time()})
        return self

    def log_artifact(self, path: str) -> "Run":
        self.artifacts.append(path)
        return self

    def add_tag(self, tag: str) -> "Run":
        if tag not in self.tags:
            self.tags.append(tag)
        return self

    def metric_history(self, key: str) -> List[float]:
        return [m["value"] for m in self.metrics if m["key"] == key]

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.__dict__)

    def save(self, directory: str) -> str:
        os.makedirs(directory, exist_ok=True)
        path = os.path.join(directory, f"{self.run_id}.json")
        with open(path, "w") as f:
            json.dump(self.to_dict(), f, default=str)
        return path

    @classmethod
    def load(cls, path: str) -> "Run":
        with open(path) as f:
            d = json.load(f)
        r = cls(d["experiment_name"], d["run_id"], d["params"])
        r.__dict__.update(d)
        return r


class Streamer:
    """Receiver of generated tokens: the generation loop calls ``put`` per token and ``end`` once
    (reference: interface_bindings/generation.py:139). This base class discards everything."""

    def put(self, token_id: int):
        pass

    def put_text(self, text: str):
        pass

    def end(self):
        pass


class TextStreamer(Streamer):
    """Decodes tokens as they arrive and hands each new piece of text to ``print_fn``. Text is re-decoded from all
    tokens so far, so multi-token characters come out whole."""

    def __init__(self, tokenizer, skip_prompt: bool = True, print_fn: Callable = print):
        self.tokenizer, self.skip_prompt, self.print_fn = tokenizer, skip_prompt, print_fn
        self._ids: List[int] = []
        self._shown = 0

    def put(self, token_id: int):
        self._ids.append(int(token_id))
        text = self.tokenizer.decode(self._ids)
        if text.endswith("�"):
            return
        if len(text) > self._shown:
            self.print_fn(text[self._shown:])
            self._shown = len(text)

    def put_text(self, text: str):
        if not self.skip_prompt:
            self.print_fn(text)

    def end(self):
        self._ids, self._shown = [], 0


class ApiKeyManager:
    """Keys with a name, a tier and an optional expiry on top of a key store; validations are cached for
    ``cache_ttl`` seconds (reference: interface_bindings/api_key_manager.py:25). Only SHA-256 digests of keys are
    kept; the raw key is returned once, by ``create_key``."""

    TIERS = {"free": 60, "pro": 600, "enterprise": 6000}

    def __init__(self, store: Optional[_svc.ApiKeyStore] = None, cache_ttl: float = 60.0, clock: Callable[[], float] = time.time):
        self.store = store or _svc.ApiKeyStore()
        self.cache_ttl, self._clock = cache_ttl, clock
        self._meta: Dict[str, dict] = {}            # key id -> record
        self._by_digest: Dict[str, str] = {}        # sha256(raw) -> key id
        self._raw: Dict[str, str] = {}              # key id -> raw key (needed to revoke in the store)
        self._cache: Dict[str, Tuple[float, dict]] = {}
        self._admin: Optional[bytes] = None

    @staticmethod
    def _digest(raw: str) -> str:
        return _crypto.sha256(raw.encode()).hex()

    def set_admin_key(self, key: str):
        self._admin = self._digest(key).encode()

    def is_admin_key(self, raw_key: str) -> bool:
        return self._admin is not None and _crypto.ct_equal(self._digest(raw_key).encode(), self._admin)

    def create_key(self, name: str = "", tier: str = "free", expires_in_days: Optional[float] = None,
                   user_id: Optional[str] = None) -> Dict[str, Any]:
        if tier not in self.TIERS:
            raise ValueError(f"unknown tier {tier!r}")
        raw = self.store.create(user_id or name or "anonymous")
        kid = uuid.uuid4().hex[:16]
        rec = {"id": kid, "name": name, "tier": tier, "rate_limit_rpm": self.TIERS[tier], "user_id": user_id, "active": True,
               "created": self._clock(), "expires": None if expires_in_days is None else self._clock() + expires_in_days * 86400.0,
               "prefix": raw[:8]}
        self._meta[kid], self._by_digest[self._digest(raw)], self._raw[kid] = rec, kid, raw
        return {**rec, "key": raw}

    def validate_key(self, raw_key: str) -> Optional[Dict[str, Any]]:
        d, now = self._digest(raw_key), self._clock()
        hit = self._cache.get(d)
        if hit and now - hit[0] < self.cache_ttl:
            rec = hit[1]
        else:
            kid = self._by_digest.get(d)
            rec = self._meta.get(kid) if kid and self.store.check(raw_key) else None
            if rec is not None:
                self._cache[d] = (now, rec)
        if rec is None or not rec["active"] or (rec["expires"] is not None and now >= rec["expires"]):
            return None
        return dict(rec)

    def revoke_key(self, key_id: str) -> bool:
        rec = self._meta.get(key_id)
        if rec is None or not rec["active"]:
            return False
        rec["active"] = False
        self.store.revoke(self._raw.pop(key_id))
        self._cache = {d: v for d, v in self._cache.items() if v[1]["id"] != key_id}
        return True

    def list_keys(self, include_inactive: bool = False) -> List[Dict[str, Any]]:
        return [dict(r) for r in self._meta.values() if include_inactive or r["active"]]


# ------------------------------------------------------------------------------------------------ audit storage
import abc  # noqa: E402
import enum  # noqa: E402
import gzip  # noqa: E402


class Severity(enum.Enum):
    """Severity scale of vulnerability findings (reference: interface_bindings/container_security.py:23); the audit
    log's own scale is ``AuditSeverity``."""

    CRITICAL = "critical"
    HIGH = "high"
    MEDIUM = "medium"
    LOW = "low"
    INFO = "info"

    @classmethod
    def from_cvss(cls, score: float) -> "Severity":
        return cls.CRITICAL if score >= 9.0 else cls.HIGH if score >= 7.0 else cls.MEDIUM if score >= 4.0 else \
            cls.LOW if score > 0.0 else cls.INFO


class AuditBackend(abc.ABC):
    """Where audit events are kept (reference: interface_bindings/audit_logger.py:207)."""

    @abc.abstractmethod
    def write(self, event) -> bool:
        ...

    @abc.abstractmethod
    def query(self, start_time=None, end_time=None, action=None, actor=None, severity=None, limit: int = 1000) -> List[dict]:
        ...

    def close(self):
        pass


class FileAuditBackend(AuditBackend):
    """JSON-lines files in ``log_dir`` with size-based rotation: when the current file passes ``max_file_size`` it is
    closed (gzip-compressed when ``compress``) and a new one is started; at most ``max_files`` rotated files are
    kept (reference: interface_bindings/audit_logger.py:231). Each line carries the SHA-256 of the previous line, so
    ``verify_chain`` finds a removed or edited record."""

    def __init__(self, log_dir: str = "audit", max_file_size: int = 100 * 1024 * 1024, max_files: int = 10, compress: bool = True):
        self.log_dir, self.max_file_size, self.max_files, self.compress = log_dir, int(max_file_size), int(max_files), compress
        os.makedirs(log_dir, exist_ok=True)
        self._lock = threading.Lock()
        self._prev = "0" * 64
        self._f = None
        self._open_new_file()

    def _current(self) -> str:
        return os.path.join(self.log_dir, "audit.jsonl")

    def _open_new_file(self):
        if self._f:
            self._f.close()
        self._f = open(self._current(), "a")

    def _rotate(self):
        self._f.close()
        stamp = f"{time.time():.6f}".replace(".", "")
        dest = os.path.join(self.log_dir, f"audit-{stamp}.jsonl")
        os.replace(self._current(), dest)
        if self.compress:
            with open(dest, "rb") as src, gzip.open(dest + ".gz", "wb") as dst:
                dst.write(src.read())
            os.remove(dest)
        old = sorted(f for f in os.listdir(self.log_dir) if f.startswith("audit-"))
        for f in old[: max(0, len(old) - self.max_files)]:
            os.remove(os.path.join(self.log_dir, f))
        self._f = open(self._current(), "a")

    @staticmethod
    def _plain(v):
        return v.value if isinstance(v, enum.Enum) else v

    def write(self, event) -> bool:
        rec = {k: self._plain(v) for k, v in (asdict(event) if hasattr(event, "__dataclass_fields__") else dict(event)).items()}
        rec.setdefault("timestamp", time.time())
        with self._lock:
            rec["prev"] = self._prev
            line = json.dumps(rec, sort_keys=True, default=str)
            self._prev = _crypto.sha256(line.encode()).hex()
            self._f.write(line + "\n")
            self._f.flush()
            if self._f.tell() >= self.max_file_size:
                self._rotate()
        return True

    def _files(self) -> List[str]:
        rotated = sorted(f for f in os.listdir(self.log_dir) if f.startswith("audit-"))
        return [os.path.join(self.log_dir, f) for f in rotated] + [self._current()]

    def _lines(self):
        for path in self._files():
            opener = gzip.open if path.endswith(".gz") else open
            try:
                with opener(path, "rt") as f:
                    yield from (l.rstrip("\n") for l in f if l.strip())
            except FileNotFoundError:
                continue

    def query(self, start_time=None, end_time=None, action=None, actor=None, severity=None, limit: int = 1000) -> List[dict]:
        out = []
        with self._lock:
            self._f.flush()
            for line in self._lines():
                r = json.loads(line)
                if start_time is not None and r["timestamp"] < start_time or end_time is not None and r["timestamp"] > end_time:
                    continue
                if action is not None and r.get("action") != self._plain(action):
                    continue
                if actor is not None and r.get("actor") != actor:
                    continue
                if severity is not None and r.get("severity") != self._plain(severity):
                    continue
                out.append(r)
        return out[-limit:]

    def verify_chain(self) -> bool:
        """True when every kept record names the hash of the record before it (the oldest kept one is the anchor)."""
        prev = None
        with self._lock:
            self._f.flush()
            for line in self._lines():
                if prev is not None and json.loads(line)["prev"] != prev:
                    return False
                prev = _crypto.sha256(line.encode()).hex()
        return True

    def close(self):
        with self._lock:
            if self._f:
                self._f.close()
                self._f = None


# ------------------------------------------------------------------------------------------------ updates
class SignedUpdate:
    """Ed25519-signed update packages with an apply / rollback state machine
    (reference: interface_bindings/secure_updates.py:18). An update is registered with its package bytes' SHA-256,
    signature and signer key; ``apply`` verifies both before marking it applied."""

    def __init__(self):
        self._updates: Dict[str, dict] = {}
        self.history: List[str] = []

    @staticmethod
    def hash_package(data: bytes) -> str:
        return _crypto.sha256(data).hex()

    @staticmethod
    def sign_update(data: bytes, signing_key: bytes) -> Tuple[bytes, bytes]:
        """(signature, public key) for ``data`` under the 32-byte Ed25519 seed ``signing_key``."""
        return _crypto.ed25519_sign(signing_key, data), _crypto.ed25519_public_key(signing_key)

    @staticmethod
    def verify_signature(data: bytes, signature: bytes, public_key: bytes) -> bool:
        return len(signature) == 64 and len(public_key) == 32 and _crypto.ed25519_verify(public_key, data, signature)

    def register_update(self, update_id: str, metadata: dict) -> None:
        """``metadata``: ``data`` (bytes), ``signature``, ``public_key``, optional ``sha256`` and ``version``."""
        self._updates[update_id] = {**metadata, "status": "pending"}

    def apply(self, update_id: str) -> bool:
        u = self._updates.get(update_id)
        if u is None or u["status"] == "applied":
            return False
        ok = self.verify_signature(u.get("data", b""), u.get("signature", b""), u.get("public_key", b""))
        if ok and "sha256" in u:
            ok = u["sha256"] == self.hash_package(u["data"])
        u["status"] = "applied" if ok else "failed"
        if ok:
            self.history.append(update_id)
        return ok

    def rollback(self, update_id: str) -> bool:
        u = self._updates.get(update_id)
        if u is None or u["status"] != "applied":
            return False
        u["status"] = "rolled_back"
        self.history.remove(update_id)
        return True

    def status(self, update_id: str) -> Optional[str]:
        u = self._updates.get(update_id)
        return u["status"] if u else None


# ------------------------------------------------------------------------------------------------ layers, losses, data
class Dense(torch.nn.Module):
    """Keras-style fully connected layer: the input width is taken from the first batch (or ``input_shape``), an
    optional activation by name follows the product (reference: interface_bindings/keras_api.py:97). On CUDA bf16
    the product and a relu / gelu / silu activation run as one tensor-core GEMM with a fused epilogue."""

    ACTIVATIONS = {None: None, "linear": None, "relu": torch.relu, "gelu": torch.nn.functional.gelu, "silu": torch.nn.functional.silu,
                   "tanh": torch.tanh, "sigmoid": torch.sigmoid, "softmax": lambda x: torch.softmax(x, -1)}

    def __init__(self, units: int, activation: Optional[str] = None, use_bias: bool = True, input_shape: Optional[Sequence[int]] = None,
                 dtype=torch.float32, device=None):
        super().__init__()
        if activation not in self.ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r}")
        self.units, self.activation, self.use_bias, self._dtype, self._device = int(units), activation, use_bias, dtype, device
        self.weight = self.bias = None
        if input_shape is not None:
            self.build(int(input_shape[-1]))

    def build(self, in_features: int):
        w = torch.empty(self.units, in_features, dtype=self._dtype, device=self._device)
        torch.nn.init.xavier_uniform_(w)
        self.weight = torch.nn.Parameter(w)
        self.bias = torch.nn.Parameter(torch.zeros(self.units, dtype=self._dtype, device=self._device)) if self.use_bias else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.weight is None:
            self._device = self._device or x.device
            self.build(x.shape[-1])
        if x.is_cuda and x.dtype == torch.bfloat16 and self.activation in (None, "linear", "relu", "gelu", "silu"):
            from .ops.gemm import gemm
            act = None if self.activation in (None, "linear") else self.activation
            return gemm(x.reshape(-1, x.shape[-1]), self.weight, bias=self.bias, act=act).view(*x.shape[:-1], self.units)
        y = torch.nn.functional.linear(x, self.weight, self.bias)
        fn = self.ACTIVATIONS[self.activation]
        return y if fn is None else fn(y)


class MAELoss:
    """Mean absolute error as a callable (reference: interface_bindings/train.py:283)."""

    def __call__(self, pred: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        return (pred.float() - target.float()).abs().mean()


class TextDataset(torch.utils.data.Dataset):
    """In-memory texts tokenised on access into fixed-length (input, target) pairs, target = input shifted by one
    (reference: interface_bindings/data.py:40). The memory-mapped token dataset is ``MemoryMappedTextDataset``."""

    def __init__(self, texts: List[str], tokenizer, max_length: int = 512, pad_id: int = 0):
        self.texts, self.tokenizer, self.max_length, self.pad_id = list(texts), tokenizer, int(max_length), pad_id

    def __len__(self) -> int:
        return len(self.texts)

    def __getitem__(self, idx):
        ids = list(self.tokenizer.encode(self.texts[idx]))[: self.max_length + 1]
        ids += [self.pad_id] * (self.max_length + 1 - len(ids))
        t = torch.tensor(ids, dtype=torch.long)
        return t[:-1], t[1:]


# ------------------------------------------------------------------------------------------------ obfuscation pass
class CfgFlattening:
    """Control-flow flattening as a pass object: every basic block of a routine becomes a case of one dispatcher loop
    keyed by a state register, so the original branch structure no longer shows in the graph
    (reference: security/obfuscation/cfg_flatten.cpp). ``apply`` takes the routine's source in the obfuscation VM's
    register IR, or an ``ObfuscatedRoutine``, and returns the flattened routine; its results are unchanged."""

    def __init__(self, seed: int = 0):
        self.seed = seed

    def apply(self, routine):
        from .security.obfuscation import ObfuscatedRoutine
        r = ObfuscatedRoutine(routine) if isinstance(routine, str) else routine
        return r.flatten(self.seed)

    __call__ = apply

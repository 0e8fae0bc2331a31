"""Logging, profiling and experiment tracking.

``Logger``: 6 levels, ANSI or JSON-lines output, per-rank prefix (include/neural_core/kernel/logger.h:28-116).
``Profiler``: named-entry aggregation (calls / total / min / max / avg), range push / pop stack, JSON export, CUDA-event
kernel timer, NVTX ranges when available (include/neural_core/kernel/profiler.h, interface_bindings/profiler.py:20-192).
``ExperimentTracker``: JSON run directories plus W&B / MLflow / composite shells (experiment_tracker.py:180-411)."""
from __future__ import annotations

import contextlib
import json
import os
import sys
import time
from collections import defaultdict
from typing import Any, Dict, List, Optional

import torch

LEVELS = {"trace": 0, "debug": 1, "info": 2, "warn": 3, "error": 4, "fatal": 5}
_COLORS = {"trace": "\033[90m", "debug": "\033[36m", "info": "\033[32m", "warn": "\033[33m", "error": "\033[31m",
           "fatal": "\033[35m"}


class Logger:
    def __init__(self, name="sneppx", level="info", json_file: Optional[str] = None, rank: Optional[int] = None,
                 stream=None, color: Optional[bool] = None):
        self.name, self.level, self.rank = name, LEVELS[level], rank if rank is not None else int(os.environ.get("RANK", 0))
        self.stream = stream or sys.stderr
        self.color = self.stream.isatty() if color is None else color
        self.json_file = open(json_file, "a") if json_file else None

    def log(self, level: str, msg: str, **fields):
        if LEVELS[level] < self.level:
            return
        ts = time.time()
        if self.json_file:
            self.json_file.write(json.dumps({"ts": ts, "level": level, "rank": self.rank, "logger": self.name, "msg": msg,
                                             **fields}) + "\n")
            self.json_file.flush()
        pre = f"[{time.strftime('%H:%M:%S', time.localtime(ts))}] [{level.upper():5}] [rank {self.rank}] "
        if self.color:
            pre = _COLORS[level] + pre + "\033[0m"
        extra = " ".join(f"{k}={v}" for k, v in fields.items())
        print(pre + msg + (" " + extra if extra else ""), file=self.stream)

    def __getattr__(self, name):
        if name in LEVELS:
            return lambda msg, **f: self.log(name, msg, **f)
        raise AttributeError(name)


class Timer:
    def __enter__(self):
        self.t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        self.elapsed = time.perf_counter() - self.t0


class Profiler:
    def __init__(self, use_nvtx: bool = True):
        self.entries: Dict[str, Dict[str, float]] = defaultdict(lambda: {"calls": 0, "total": 0.0, "min": float("inf"), "max": 0.0})
        self._stack: List[tuple] = []
        self.use_nvtx = use_nvtx and torch.cuda.is_available()

    def _add(self, name, dt):
        e = self.entries[name]
        e["calls"] += 1
        e["total"] += dt
        e["min"] = min(e["min"], dt)
        e["max"] = max(e["max"], dt)

    def range_push(self, name):
        if self.use_nvtx:
            torch.cuda.nvtx.range_push(name)
        self._stack.append((name, time.perf_counter()))

    def range_pop(self):
        name, t0 = self._stack.pop()
        if self.use_nvtx:
            torch.cuda.nvtx.range_pop()
        self._add(name, time.perf_counter() - t0)

    @contextlib.contextmanager
    def range(self, name):
        self.range_push(name)
        try:
            yield
        finally:
            self.range_pop()

    @contextlib.contextmanager
    def kernel(self, name):
        """Device time of the enclosed launches (two CUDA events + sync), like SNEPPX_PROFILE_KERNEL."""
        if not torch.cuda.is_available():
            with self.range(name):
                yield
            return
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        yield
        e1.record()
        e1.synchronize()
        self._add(name, e0.elapsed_time(e1) / 1e3)

    def summary(self):
        return {k: {**v, "avg": v["total"] / max(1, v["calls"])} for k, v in self.entries.items()}

    def export_json(self, path):
        with open(path, "w") as f:
            json.dump(self.summary(), f, indent=2)

    def report(self) -> str:
        rows = sorted(self.summary().items(), key=lambda kv: -kv[1]["total"])
        return "\n".join(f"{k:32s} calls {v['calls']:6d} total {v['total']*1e3:10.3f} ms avg {v['avg']*1e3:9.3f} ms"
                         for k, v in rows)


def timeit(fn):
    def wrapped(*a, **k):
        t0 = time.perf_counter()
        out = fn(*a, **k)
        wrapped.last = time.perf_counter() - t0
        return out
    wrapped.last = 0.0
    return wrapped


class MemoryTracker:
    def snapshot(self):
        if torch.cuda.is_available():
            return {"allocated": torch.cuda.memory_allocated(), "reserved": torch.cuda.memory_reserved(),
                    "peak": torch.cuda.max_memory_allocated()}
        import resource
        return {"rss_kb": resource.getrusage(resource.RUSAGE_SELF).ru_maxrss}


def estimate_flops(cfg, tokens: int, training: bool = True) -> float:
    """6 * params * tokens for training (2 * for inference) plus the attention term."""
    n = cfg.estimate_parameters() - cfg.vocab_size * cfg.hidden_size * (0 if cfg.tie_word_embeddings else 1)
    return (6 if training else 2) * n * tokens


class ExperimentTracker:
    """Local JSON runs directory: runs/<run_id>/{params.json, metrics.jsonl, artifacts/}."""

    def __init__(self, directory="runs", experiment="default"):
        self.dir, self.experiment, self.run_dir, self._f = directory, experiment, None, None

    def start_run(self, run_name: Optional[str] = None, params: Optional[dict] = None):
        rid = run_name or time.strftime("%Y%m%d-%H%M%S")
        self.run_dir = os.path.join(self.dir, self.experiment, rid)
        os.makedirs(os.path.join(self.run_dir, "artifacts"), exist_ok=True)
        if params:
            self.log_params(params)
        self._f = open(os.path.join(self.run_dir, "metrics.jsonl"), "a")
        return rid

    def log_params(self, params: dict):
        with open(os.path.join(self.run_dir, "params.json"), "w") as f:
            json.dump(params, f, indent=2, default=str)

    def log_metrics(self, metrics: Dict[str, Any], step: Optional[int] = None):
        self._f.write(json.dumps({"step": step, "ts": time.time(), **{k: float(v) for k, v in metrics.items()}}) + "\n")
        self._f.flush()

    def log_artifact(self, path: str):
        import shutil
        shutil.copy(path, os.path.join(self.run_dir, "artifacts"))

    def end_run(self):
        if self._f:
            self._f.close()
            self._f = None


class WandbTracker(ExperimentTracker):
    """Weights & Biases. With the ``wandb`` package importable the run is also opened there in offline mode; in every
    case an offline-run directory in wandb's layout is written (``wandb/offline-run-<time>-<id>/files`` with
    ``config.yaml``, ``wandb-history.jsonl`` - one JSON object per logged step with ``_step`` / ``_timestamp`` /
    ``_runtime`` - and ``wandb-summary.json`` holding the last value of every metric), next to the local files."""

    def start_run(self, run_name=None, params=None):
        import secrets
        try:
            import wandb  # noqa: F401
            os.makedirs(self.dir, exist_ok=True)
            self._wandb = wandb.init(project=self.experiment, name=run_name, config=params, mode="offline", dir=self.dir)
        except Exception:  # noqa: BLE001
            self._wandb = None
        rid = super().start_run(run_name, params)
        self.wandb_id = secrets.token_hex(4)
        self._t0 = time.time()
        self.wandb_dir = os.path.join(self.dir, "wandb", f"offline-run-{time.strftime('%Y%m%d_%H%M%S')}-{self.wandb_id}", "files")
        os.makedirs(self.wandb_dir, exist_ok=True)
        with open(os.path.join(self.wandb_dir, "config.yaml"), "w") as f:
            f.write("wandb_version: 1\n\n")
            for k, v in (params or {}).items():
                f.write(f"{k}:\n  desc: null\n  value: {json.dumps(v, default=str)}\n")
        self._summary, self._wstep = {}, 0
        return rid

    def log_metrics(self, metrics, step=None):
        if getattr(self, "_wandb", None):
            self._wandb.log(metrics, step=step)
        super().log_metrics(metrics, step)
        self._wstep = step if step is not None else self._wstep + 1
        row = {k: float(v) for k, v in metrics.items()}
        now = time.time()
        row.update(_step=self._wstep, _timestamp=now, _runtime=now - self._t0)
        with open(os.path.join(self.wandb_dir, "wandb-history.jsonl"), "a") as f:
            f.write(json.dumps(row) + "\n")
        self._summary.update(row)
        with open(os.path.join(self.wandb_dir, "wandb-summary.json"), "w") as f:
            json.dump(self._summary, f)

    def end_run(self):
        if getattr(self, "_wandb", None):
            self._wandb.finish()
        super().end_run()


class MLflowTracker(ExperimentTracker):
    """Writes MLflow's file-store layout under ``<dir>/mlruns`` (what ``mlflow ui --backend-store-uri <dir>/mlruns``
    reads): ``<experiment id>/meta.yaml``, and per run ``meta.yaml``, ``params/<key>`` (the value as text),
    ``metrics/<key>`` (one ``<timestamp ms> <value> <step>`` line per logged point), ``tags/<key>`` and ``artifacts/``.
    The local JSONL files of the base tracker are written as well."""

    def _experiment_dir(self):
        root = os.path.join(self.dir, "mlruns")
        os.makedirs(root, exist_ok=True)
        for d in sorted(os.listdir(root)):
            meta = os.path.join(root, d, "meta.yaml")
            if os.path.exists(meta) and f"name: {self.experiment}\n" in open(meta).read():
                return os.path.join(root, d), d
        ids = [int(d) for d in os.listdir(root) if d.isdigit()]
        eid = str(max(ids) + 1 if ids else 0)
        path = os.path.join(root, eid)
        os.makedirs(path)
        with open(os.path.join(path, "meta.yaml"), "w") as f:
            f.write(f"artifact_location: {path}\ncreation_time: {int(time.time() * 1000)}\nexperiment_id: '{eid}'\n"
                    f"last_update_time: {int(time.time() * 1000)}\nlifecycle_stage: active\nname: {self.experiment}\n")
        return path, eid

    def start_run(self, run_name=None, params=None):
        import uuid
        rid = super().start_run(run_name, None)
        exp_dir, eid = self._experiment_dir()
        self.mlflow_run_id = uuid.uuid4().hex
        self.mlflow_dir = os.path.join(exp_dir, self.mlflow_run_id)
        for sub in ("params", "metrics", "tags", "artifacts"):
            os.makedirs(os.path.join(self.mlflow_dir, sub))
        self._start_ms = int(time.time() * 1000)
        self._write_meta("RUNNING", None)
        self.set_tags({"mlflow.runName": rid, "mlflow.source.type": "LOCAL", "mlflow.user": os.environ.get("USER", "unknown")})
        self._eid = eid
        if params:
            self.log_params(params)
        return rid

    def _write_meta(self, status, end_ms):
        names = {"RUNNING": 1, "FINISHED": 3, "FAILED": 4}
        with open(os.path.join(self.mlflow_dir, "meta.yaml"), "w") as f:
            f.write(f"artifact_uri: {os.path.join(self.mlflow_dir, 'artifacts')}\nend_time: {end_ms if end_ms else 'null'}\n"
                    f"entry_point_name: ''\nexperiment_id: '{getattr(self, '_eid', '0')}'\nlifecycle_stage: active\n"
                    f"run_id: {self.mlflow_run_id}\nrun_uuid: {self.mlflow_run_id}\nsource_name: ''\nsource_type: 4\n"
                    f"source_version: ''\nstart_time: {self._start_ms}\nstatus: {names[status]}\ntags: []\nuser_id: "
                    f"{os.environ.get('USER', 'unknown')}\n")

    @staticmethod
    def _safe_key(k: str) -> str:
        import re
        return re.sub(r"[^A-Za-z0-9_./ -]", "_", str(k)).strip("/").replace("..", "_") or "_"

    def set_tags(self, tags: dict):
        for k, v in tags.items():
            path = os.path.join(self.mlflow_dir, "tags", self._safe_key(k))
            os.makedirs(os.path.dirname(path), exist_ok=True)
            with open(path, "w") as f:
                f.write(str(v))

    def log_params(self, params: dict):
        super().log_params(params)
        for k, v in params.items():
            path = os.path.join(self.mlflow_dir, "params", self._safe_key(k))
            os.makedirs(os.path.dirname(path), exist_ok=True)
            with open(path, "w") as f:
                f.write(str(v))

    def log_metrics(self, metrics, step=None):
        super().log_metrics(metrics, step)
        ts = int(time.time() * 1000)
        for k, v in metrics.items():
            path = os.path.join(self.mlflow_dir, "metrics", self._safe_key(k))
            os.makedirs(os.path.dirname(path), exist_ok=True)
            with open(path, "a") as f:
                f.write(f"{ts} {float(v)} {int(step) if step is not None else 0}\n")

    def log_artifact(self, path: str):
        import shutil
        super().log_artifact(path)
        shutil.copy(path, os.path.join(self.mlflow_dir, "artifacts"))

    def end_run(self, status: str = "FINISHED"):
        super().end_run()
        self._write_meta(status, int(time.time() * 1000))

    def read_metric(self, key: str):
        """[(timestamp ms, value, step)] of one metric of the current run, as stored."""
        with open(os.path.join(self.mlflow_dir, "metrics", self._safe_key(key))) as f:
            return [(int(a), float(b), int(c)) for a, b, c in (line.split() for line in f if line.strip())]


class TensorBoardTracker(ExperimentTracker):
    """TensorBoard event files, written directly (TFRecord framing with masked CRC-32C, ``Event`` / ``Summary`` protobuf
    messages encoded by hand), so that ``tensorboard --logdir <directory>`` shows the run without TensorFlow or the
    ``tensorboard`` package being importable where training runs. Scalars become ``simple_value`` summaries, parameters a
    text summary (``text`` plugin, markdown table), histograms ``HistogramProto`` values. The JSON files of the base
    class are written too. The reference's run tracker keeps ``metadata.json`` + ``metrics.jsonl`` only and points to
    TensorBoard's ``runs/`` layout as its model (bindings/python/SneppX_ALG/interface_bindings/experiment.py:1-18)."""

    _CRC_TABLE = None

    @classmethod
    def _crc32c(cls, data: bytes) -> int:
        if cls._CRC_TABLE is None:
            table = []
            for i in range(256):
                c = i
                for _ in range(8):
                    c = (c >> 1) ^ 0x82F63B78 if c & 1 else c >> 1
                table.append(c)
            cls._CRC_TABLE = table
        crc = 0xFFFFFFFF
        for b in data:
            crc = cls._CRC_TABLE[(crc ^ b) & 0xFF] ^ (crc >> 8)
        return crc ^ 0xFFFFFFFF

    @classmethod
    def _masked_crc(cls, data: bytes) -> int:
        c = cls._crc32c(data)
        return ((((c >> 15) | (c << 17)) & 0xFFFFFFFF) + 0xA282EAD8) & 0xFFFFFFFF

    @staticmethod
    def _varint(v: int) -> bytes:
        v &= (1 << 64) - 1
        out = bytearray()
        while True:
            out.append((v & 0x7F) | (0x80 if v > 0x7F else 0))
            v >>= 7
            if not v:
                return bytes(out)

    @classmethod
    def _field(cls, number: int, wire: int, payload: bytes) -> bytes:
        key = cls._varint((number << 3) | wire)
        return key + (cls._varint(len(payload)) + payload if wire == 2 else payload)

    @classmethod
    def _event(cls, wall_time: float, step: int = 0, file_version: Optional[str] = None, summary: Optional[bytes] = None) -> bytes:
        import struct
        msg = cls._field(1, 1, struct.pack("<d", wall_time)) + cls._field(2, 0, cls._varint(step))
        if file_version is not None:
            msg += cls._field(3, 2, file_version.encode())
        if summary is not None:
            msg += cls._field(5, 2, summary)
        return msg

    def _write_event(self, event: bytes) -> None:
        import struct
        head = struct.pack("<Q", len(event))
        self._tb.write(head + struct.pack("<I", self._masked_crc(head)) + event + struct.pack("<I", self._masked_crc(event)))
        self._tb.flush()

    def start_run(self, run_name=None, params=None):
        import socket
        rid = super().start_run(run_name, None)
        name = f"events.out.tfevents.{int(time.time())}.{socket.gethostname()}.{os.getpid()}.0"
        self._tb = open(os.path.join(self.run_dir, name), "ab")
        self._write_event(self._event(time.time(), 0, file_version="brain.Event:2"))
        if params:
            self.log_params(params)
        return rid

    def log_params(self, params: dict):
        super().log_params(params)
        rows = "".join(f"| {k} | {v} |\n" for k, v in sorted(params.items()))
        text = ("| parameter | value |\n|---|---|\n" + rows).encode()
        # TensorProto{dtype=DT_STRING(7), tensor_shape{dim{size=1}}, string_val=[text]}; metadata names the text plugin
        tensor = self._field(1, 0, self._varint(7)) + self._field(2, 2, self._field(2, 2, self._field(1, 0, self._varint(1)))) \
            + self._field(8, 2, text)
        meta = self._field(1, 2, self._field(1, 2, b"text"))
        value = self._field(1, 2, b"parameters/text_summary") + self._field(9, 2, meta) + self._field(8, 2, tensor)
        self._write_event(self._event(time.time(), 0, summary=self._field(1, 2, value)))

    def log_metrics(self, metrics, step=None):
        import struct
        super().log_metrics(metrics, step)
        values = b"".join(self._field(1, 2, self._field(1, 2, str(k).encode()) + self._field(2, 5, struct.pack("<f", float(v))))
                          for k, v in metrics.items())
        self._write_event(self._event(time.time(), int(step or 0), summary=values))

    def log_histogram(self, tag: str, values, step: int = 0, bins: int = 30):
        """A histogram of ``values`` (tensor, array or list) under ``tag``."""
        import struct
        import numpy as np
        v = np.asarray(values.detach().float().cpu().numpy() if hasattr(values, "detach") else values, dtype=np.float64).ravel()
        if v.size == 0:
            return
        counts, edges = np.histogram(v, bins=bins)
        packed = lambda arr: struct.pack(f"<{len(arr)}d", *[float(x) for x in arr])
        histo = b"".join(self._field(i, 1, struct.pack("<d", x)) for i, x in
                         ((1, v.min()), (2, v.max()), (3, float(v.size)), (4, v.sum()), (5, float((v * v).sum())))) \
            + self._field(6, 2, packed(edges[1:])) + self._field(7, 2, packed(counts))
        value = self._field(1, 2, tag.encode()) + self._field(5, 2, histo)
        self._write_event(self._event(time.time(), int(step), summary=self._field(1, 2, value)))

    def end_run(self):
        super().end_run()
        if getattr(self, "_tb", None):
            self._tb.close()
            self._tb = None


class CompositeTracker:
    def __init__(self, trackers):
        self.trackers = list(trackers)

    def __getattr__(self, name):
        def fan(*a, **k):
            return [getattr(t, name)(*a, **k) for t in self.trackers][0]
        return fan


def make_tracker(kind="local", **kw):
    return {"local": ExperimentTracker, "wandb": WandbTracker, "mlflow": MLflowTracker,
            "tensorboard": TensorBoardTracker}.get(kind, ExperimentTracker)(**kw)



def bench_marker(text: str):
    """``[BENCH] <text>`` on stderr when the environment has ``SNEPPX_BENCH=1``: the start / done markers that the
    reference's HSS and SER forwards print for its external bench tool (algorithms/hss/core/forward.c:143,174,
    algorithms/ser/core/forward_layer.c:32). Silent otherwise, so that training loops pay one dictionary lookup."""
    import os
    import sys
    if os.environ.get("SNEPPX_BENCH") == "1":
        print(f"[BENCH] {text}", file=sys.stderr, flush=True)


def parse_bench_markers(stderr_text: str):
    """Pairs ``[BENCH] X start`` / ``[BENCH] X done`` lines of a captured stderr into [(X, count)] in first-seen order."""
    seen, order = {}, []
    for line in stderr_text.splitlines():
        if line.startswith("[BENCH] ") and line.endswith(" done"):
            name = line[8:-5]
            if name not in seen:
                order.append(name)
            seen[name] = seen.get(name, 0) + 1
    return [(n, seen[n]) for n in order]

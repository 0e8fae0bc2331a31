"""Second half of the reference's flat namespace: service singletons and their module-level helpers (audit log, DDoS
mitigation, key manager, usage tracker, user store, container security), serving schema records, the evaluation
harness, experiment store, ONNX / graph / NPE / ARC class aliases, data and tokenizer aliases, privacy mechanisms,
thread pools, streamers and the ``*_kernel`` entry points (``cuda_kernels.py``) mapped onto this package's ops.
``SneppX_ALG`` resolves names here after ``compat``.

Not reproduced, by design (one CUDA sm_100a device layer, portable C++ host code): the multi-vendor back-end and
driver tables (``NPUBackend``, ``OpenVINOBackend``, ``ROCmDriver``, ``TPUDriver``, ``TensorRTExporter``, ``AutoBackend``
...) and the x86 assembly wrappers (``AESNI``, ``SHANI``, ``Poly1305ASM``, ``Ed25519ASM``, ``ChaCha20AVX2``,
``FirewallASM``, ``Asm*``).
"""
from __future__ import annotations

import enum
import json
import os
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence

import torch

from .algorithms import arc as _arc
from .algorithms import fm as _fm
from .algorithms import npe as _npe
from .onnx import toolkit as _onnx
from .security import services as _svc
from .training import data as _data

# ----------------------------------------------------------------------------------------- service singletons
_singletons: Dict[str, Any] = {}


def _accessor(key: str, factory: Callable[[], Any]):
    def get():
        if key not in _singletons:
            _singletons[key] = factory()
        return _singletons[key]

    def set_(obj):
        _singletons[key] = obj
        return obj
    return get, set_


get_audit_logger, set_audit_logger = _accessor("audit", lambda: _svc.AuditLogger(os.path.join(os.path.expanduser("~/.sneppx"), "audit.log")))
get_ddos_mitigation, set_ddos_mitigation = _accessor("ddos", _svc.DDoSMitigator)
get_key_manager, set_key_manager = _accessor("keys", _svc.ApiKeyStore)
get_usage_tracker, set_usage_tracker = _accessor("usage", _svc.UsageTracker)
DDoSMitigation = _svc.DDoSMitigator


class SelfAuditor:
    """Configuration audit with a score: ``audit(config)`` lists findings, ``score`` is the share of checks passed."""

    CHECKS = 4

    def __init__(self):
        self.findings: List[str] = []

    def audit(self, config: dict) -> List[str]:
        self.findings = _svc.self_audit(config)
        return self.findings

    @property
    def score(self) -> float:
        return 1.0 - len(self.findings) / self.CHECKS


class NetworkFuzzer:
    """Mutation fuzzer bound to a seed corpus; ``run(target)`` returns the crashing inputs of this campaign."""

    def __init__(self, seeds: Sequence[bytes], iterations: int = 200, seed: int = 0):
        self.seeds, self.iterations, self.seed = list(seeds), iterations, seed
        self.crashes: List[dict] = []

    def run(self, target: Callable[[bytes], None]) -> List[dict]:
        self.crashes = _svc.fuzz(target, self.seeds, self.iterations, self.seed)
        return self.crashes


class LTLProperty:
    """A named temporal property. ``holds_on(trace)`` evaluates it on one finite trace of labelled states;
    ``holds_in(model)`` checks every infinite run of a ``security.formal.FormalModel``."""

    def __init__(self, formula, name: str = ""):
        from .security.formal import parse_ltl
        self.formula = parse_ltl(formula) if isinstance(formula, str) else formula
        self.name = name or str(formula)

    def holds_on(self, trace: List[dict]) -> bool:
        return _svc.ltl_check(self._finite(self.formula), trace)

    @staticmethod
    def _finite(f):
        if f is True or f is False or f[0] in ("ap",):
            return ("ap", "__true__") if f is True else (("not", ("ap", "__true__")) if f is False else f)
        if f[0] == "implies":
            return ("or", ("not", LTLProperty._finite(f[1])), LTLProperty._finite(f[2]))
        if f[0] == "release":      # f R g on a finite trace: g holds up to and including the first f (or to the end)
            a, b = LTLProperty._finite(f[1]), LTLProperty._finite(f[2])
            return ("or", ("always", b), ("until", b, ("and", a, b)))
        return (f[0],) + tuple(LTLProperty._finite(x) if isinstance(x, tuple) or x is True or x is False else x for x in f[1:])

    def holds_in(self, model):
        return model.check_ltl(self.formula)


class ModelChecker:
    """Builds a transition system and checks properties on it (``security.formal.FormalModel`` underneath)."""

    def __init__(self):
        from .security.formal import FormalModel
        self.model = FormalModel()

    def add_state(self, state: int, props=(), initial=False, accepting=False, error=False):
        self.model.add_state(state, props, initial, accepting, error)
        return self

    def add_transition(self, a: int, b: int, label: str = ""):
        self.model.add_transition(a, b, label)
        return self

    def check(self, prop) -> bool:
        prop = prop if isinstance(prop, LTLProperty) else LTLProperty(prop)
        return bool(prop.holds_in(self.model))

    def counterexample(self, prop):
        prop = prop if isinstance(prop, LTLProperty) else LTLProperty(prop)
        return prop.holds_in(self.model).counterexample

    def deadlocks(self):
        return self.model.deadlocks()

    def reachable(self, a: int, b: int) -> bool:
        return self.model.is_reachable(a, b)


def audit_log(actor: str, action: str, **details):
    os.makedirs(os.path.expanduser("~/.sneppx"), exist_ok=True)
    return get_audit_logger().log(actor, action, **details)


def audit_login(user: str, success: bool = True, **kw):
    return audit_log(user, "login", success=success, **kw)


def audit_data_access(user: str, resource: str, **kw):
    return audit_log(user, "data_access", resource=resource, **kw)


def audit_config_change(user: str, key: str, old=None, new=None):
    return audit_log(user, "config_change", key=key, old=old, new=new)


def audit_security_event(kind: str, **kw):
    return audit_log("system", "security_event", kind=kind, **kw)


def verify_audit_chain() -> bool:
    return get_audit_logger().verify()


def check_request(client_ip: str) -> bool:
    return get_ddos_mitigation().check(client_ip)


def ban_ip(ip: str, seconds: float = 3600.0):
    d = get_ddos_mitigation()
    d.banned[ip] = d.clock() + seconds


def unban_ip(ip: str):
    get_ddos_mitigation().banned.pop(ip, None)


def get_ip_info(ip: str) -> dict:
    d = get_ddos_mitigation()
    return {"ip": ip, "banned": ip in d.banned and d.clock() < d.banned[ip], "violations": d.violations.get(ip, 0)}


def get_ddos_stats() -> dict:
    d = get_ddos_mitigation()
    return {"clients": len(d.buckets), "banned": sum(1 for t in d.banned.values() if d.clock() < t), "violations": sum(d.violations.values())}


class UserStore:
    """Username -> salted PBKDF2 password hash and roles."""

    def __init__(self):
        self.users: Dict[str, dict] = {}

    def add_user(self, name: str, password: str, roles: Sequence[str] = ("user",)):
        from .security import crypto
        salt = os.urandom(16)
        self.users[name] = {"salt": salt, "hash": crypto.pbkdf2_sha256(password.encode(), salt, 20000), "roles": list(roles)}

    def authenticate(self, name: str, password: str) -> bool:
        from .security import crypto
        u = self.users.get(name)
        return bool(u) and crypto.ct_equal(u["hash"], crypto.pbkdf2_sha256(password.encode(), u["salt"], 20000))

    def has_role(self, name: str, role: str) -> bool:
        return role in self.users.get(name, {}).get("roles", [])


get_user_store, set_user_store = _accessor("users", UserStore)


@dataclass
class SBOMComponent:
    name: str
    version: str
    vulnerable: bool = False
    cves: List[str] = field(default_factory=list)


class SBOMGenerator:
    def generate(self, packages: Dict[str, str], known_cves: Optional[Dict[str, List[str]]] = None) -> dict:
        return _svc.sbom(packages, known_cves)


class ContainerSecurityManager:
    """Requirement / image scans against a table of known-vulnerable versions."""

    def __init__(self, known_cves: Optional[Dict[str, List[str]]] = None):
        self.known, self.history = known_cves or {}, []

    def scan_requirements(self, packages: Dict[str, str]) -> dict:
        rep = _svc.sbom(packages, self.known)
        self.history.append(rep)
        return rep

    scan_image = scan_requirements


get_container_security, set_container_security = _accessor("container", ContainerSecurityManager)
generate_sbom = lambda packages, known=None: _svc.sbom(packages, known)  # noqa: E731
scan_requirements = scan_image = lambda packages: get_container_security().scan_requirements(packages)  # noqa: E731
get_scan_history = lambda: get_container_security().history  # noqa: E731
get_security, set_security = _accessor("security", lambda: {"ddos": get_ddos_mitigation(), "keys": get_key_manager()})


class SignedUpdateManager:
    """stage -> verify -> install with rollback of the previous file (signed manifests from ``security.services``)."""

    def __init__(self, key: bytes, install_dir: str):
        self.key, self.dir, self.staged = key, install_dir, None
        os.makedirs(install_dir, exist_ok=True)

    def stage_update(self, path: str, manifest: dict, min_version: str = "0") -> bool:
        ok = _svc.verify_update(path, manifest, self.key, min_version)
        self.staged = (path, manifest) if ok else None
        return ok

    def install_update(self) -> str:
        if not self.staged:
            raise RuntimeError("nothing staged")
        import shutil
        path, man = self.staged
        dst = os.path.join(self.dir, man["file"])
        if os.path.exists(dst):
            shutil.copy2(dst, dst + ".previous")
        shutil.copy2(path, dst)
        self.staged = None
        return dst

    def rollback_update(self, file_name: str) -> bool:
        dst = os.path.join(self.dir, file_name)
        if not os.path.exists(dst + ".previous"):
            return False
        os.replace(dst + ".previous", dst)
        return True




# ----------------------------------------------------------------------------------------- serving schema and helpers
@dataclass
class GenerateRequest:
    prompt: str
    max_new_tokens: int = 64
    do_sample: bool = False
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    num_beams: int = 1
    stop_strings: Optional[List[str]] = None
    model: Optional[str] = None

    def __post_init__(self):
        if not 1 <= self.max_new_tokens <= 4096:
            raise ValueError("max_new_tokens must be in 1..4096")


@dataclass
class GenerateResponse:
    generated_text: str
    token_ids: List[int]
    prompt_tokens: int
    completion_tokens: int
    total_tokens: int
    model: str
    created: int


@dataclass
class BatchGenerateRequest:
    prompts: List[str]
    max_new_tokens: int = 64
    model: Optional[str] = None


@dataclass
class BatchGenerateResponse:
    results: List[GenerateResponse]


@dataclass
class ChatCompletionRequest:
    messages: List[Dict[str, str]]
    max_tokens: int = 64
    temperature: float = 1.0
    model: Optional[str] = None


@dataclass
class ChatCompletionResponse:
    id: str
    choices: List[dict]
    usage: Dict[str, int]
    object: str = "chat.completion"


@dataclass
class HealthResponse:
    status: str = "ok"
    models: List[str] = field(default_factory=list)


@dataclass
class ModelInfo:
    id: str
    family: str = ""
    params: float = 0.0


@dataclass
class ModelListResponse:
    data: List[ModelInfo] = field(default_factory=list)


@dataclass
class GenerationConfig:
    max_new_tokens: int = 64
    do_sample: bool = False
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    num_beams: int = 1


@dataclass
class ServingConfig:
    host: str = "127.0.0.1"
    port: int = 8000
    max_batch_size: int = 32
    batch_timeout_ms: float = 2.0
    warmup_ticks: int = 0


class ServingError(RuntimeError):
    pass


@dataclass
class PagedAttentionConfig:
    block_size: int = 16
    num_blocks: int = 2048
    enable_prefix_cache: bool = True


def serve_from_config(path: str):
    """Builds the FastAPI application from a YAML / JSON file: {models: {id: preset}, default: id, api_keys: [...]}."""
    import yaml
    from .models import create_model
    from .serving.server import create_app
    cfg = yaml.safe_load(open(path)) if path.endswith((".yaml", ".yml")) else json.load(open(path))
    models = {mid: {"model": create_model(preset).eval()} for mid, preset in cfg["models"].items()}
    return create_app(models, cfg.get("default"), api_keys=set(cfg.get("api_keys") or []) or None)


inference_app = serve_from_config


from .compat_classes import Streamer  # noqa: E402


class TokenStreamer(Streamer):
    """Collects tokens pushed by a generation loop (``put(token)``) or by the engine's ``on_token`` callback
    (``put(request_id, token)``); iterating yields them as they arrive, ``get_tokens`` returns those seen so far."""

    def __init__(self):
        self._q, self._cv, self._done = [], threading.Condition(), False

    def put(self, *args):
        with self._cv:
            self._q.append(int(args[-1]))
            self._cv.notify_all()

    def get_tokens(self) -> List[int]:
        with self._cv:
            return list(self._q)

    def end(self):
        with self._cv:
            self._done = True
            self._cv.notify_all()

    def __iter__(self):
        i = 0
        while True:
            with self._cv:
                self._cv.wait_for(lambda: i < len(self._q) or self._done)
                if i >= len(self._q):
                    return
                tok = self._q[i]
            i += 1
            yield tok




def sample(logits, temperature=1.0, top_k=0, top_p=1.0, generator=None):
    from .serving.generation import sample_from_logits
    return sample_from_logits(logits, True, temperature, top_k, top_p, generator)


def paged_attention_forward(q, k_cache, v_cache, block_table, lens):
    from .ops import paged
    return paged.paged_decode(q, k_cache, v_cache, block_table, lens)


def incremental_attention_forward(q, k, v, state: Optional[dict] = None):
    """One more block of keys / values for fixed queries: returns (output, state) with the running log-sum-exp, so a
    long context can be consumed piece by piece (the NumPy reference's IncrementalAttentionState)."""
    from .ops.functional import attention_with_lse
    from .parallel.context import merge_attention_blocks
    o, lse = attention_with_lse(q, k, v, causal=False)
    if state:
        o, lse = merge_attention_blocks(state["o"], state["lse"], o, lse)
    return o.to(q.dtype), {"o": o.float(), "lse": lse}




def chunked_prefill_forward(model, input_ids, chunk: int = 512):
    """Prefill in chunks through the model's cache contract; returns the logits of the last position."""
    past, logits = None, None
    for s in range(0, input_ids.shape[1], chunk):
        out = model(input_ids[:, s:s + chunk], past_key_values=past, use_cache=True)
        past, logits = out["past_key_values"], out["logits"][:, -1]
    return logits, past


# ----------------------------------------------------------------------------------------- evaluation harness
@dataclass
class EvalResult:
    task: str
    score: float
    n: int


@dataclass
class EvalSummary:
    results: List[EvalResult]

    @property
    def mean(self) -> float:
        return sum(r.score for r in self.results) / max(len(self.results), 1)


@dataclass
class EvalConfig:
    max_new_tokens: int = 16
    batch_size: int = 8


class Task:
    name = "task"

    def __init__(self, examples: List[dict]):
        self.examples = examples

    def score(self, predict: Callable[[dict], Any]) -> EvalResult:
        ok = sum(1 for ex in self.examples if self.correct(predict(ex), ex))
        return EvalResult(self.name, ok / max(len(self.examples), 1), len(self.examples))

    def correct(self, pred, ex) -> bool:
        raise NotImplementedError


class ExactMatchTask(Task):
    name = "exact_match"

    def correct(self, pred, ex):
        return str(pred).strip() == str(ex["answer"]).strip()


class MultipleChoiceTask(Task):
    """`predict` returns the index of the chosen option (e.g. the one with the highest log-likelihood)."""
    name = "multiple_choice"

    def correct(self, pred, ex):
        return int(pred) == int(ex["label"])


class CodingTask(Task):
    """`predict` returns source text defining the function named in the example; it is run against the tests."""
    name = "coding"

    timeout_s = 10.0

    def correct(self, pred, ex):
        """Model-written code never runs inside this process: a child interpreter (isolated mode, no site
        packages, empty environment, scratch working directory) loads the source, runs the tests and prints a
        JSON verdict; a crash, a hang past ``timeout_s`` or anything but ``true`` on the last line counts as wrong."""
        import json as _json
        import subprocess
        import sys
        import tempfile
        driver = ("import json,sys\n"
                  "job=json.load(sys.stdin)\n"
                  "scope={}\n"
                  "exec(job['src'],scope)\n"
                  "f=scope[job['entry']]\n"
                  "print(json.dumps(all(f(*a)==w for a,w in job['tests'])))\n")
        try:
            job = _json.dumps({"src": str(pred), "entry": ex["entry_point"], "tests": [[list(a), w] for a, w in ex["tests"]]})
        except (TypeError, ValueError):
            return False
        try:
            with tempfile.TemporaryDirectory() as tmp:
                r = subprocess.run([sys.executable, "-I", "-S", "-c", driver], input=job, capture_output=True, text=True,
                                   timeout=self.timeout_s, cwd=tmp, env={})
        except (subprocess.TimeoutExpired, OSError):
            return False
        return r.returncode == 0 and r.stdout.strip().splitlines()[-1:] == ["true"]


class EvalHarness:
    def __init__(self, tasks: Sequence[Task], config: Optional[EvalConfig] = None):
        self.tasks, self.config = list(tasks), config or EvalConfig()

    def run(self, predict: Callable[[dict], Any]) -> EvalSummary:
        return EvalSummary([t.score(predict) for t in self.tasks])


MMLU_CATEGORIES = {"stem": ["physics", "chemistry", "biology", "computer_science", "math", "engineering"],
                   "humanities": ["history", "philosophy", "law"], "social_sciences": ["politics", "culture", "economics", "geography", "psychology"],
                   "other": ["other", "business", "health"]}


# ----------------------------------------------------------------------------------------- experiments
@dataclass
class ExperimentRun:
    run_id: str
    params: Dict[str, Any] = field(default_factory=dict)
    metrics: Dict[str, List[float]] = field(default_factory=dict)
    status: str = "running"

    def log_metric(self, name: str, value: float):
        self.metrics.setdefault(name, []).append(float(value))

    def finish(self, status: str = "finished"):
        self.status = status




class Experiment:
    def __init__(self, name: str):
        self.name, self.runs = name, []

    def start_run(self, params: Optional[dict] = None) -> ExperimentRun:
        r = ExperimentRun(f"{self.name}-{len(self.runs)}", dict(params or {}))
        self.runs.append(r)
        return r

    def best_run(self, metric: str, mode: str = "min") -> ExperimentRun:
        cands = [r for r in self.runs if r.metrics.get(metric)]
        pick = min if mode == "min" else max
        return pick(cands, key=lambda r: pick(r.metrics[metric]))


class ExperimentStore:
    """Experiments as JSON files in a directory."""

    def __init__(self, directory: str):
        self.dir = directory
        os.makedirs(directory, exist_ok=True)

    def save(self, exp: Experiment):
        with open(os.path.join(self.dir, exp.name + ".json"), "w") as f:
            json.dump({"name": exp.name, "runs": [asdict(r) for r in exp.runs]}, f)

    def load(self, name: str) -> Experiment:
        d = json.load(open(os.path.join(self.dir, name + ".json")))
        exp = Experiment(d["name"])
        exp.runs = [ExperimentRun(**r) for r in d["runs"]]
        return exp

    def list(self) -> List[str]:
        return sorted(f[:-5] for f in os.listdir(self.dir) if f.endswith(".json"))


def load_experiment(directory: str, name: str) -> Experiment:
    return ExperimentStore(directory).load(name)


def experiment_cli_main(argv=None):
    from .cli import experiment_main
    return experiment_main(argv)


class LineageStore:
    """Parent links between artefacts (datasets, checkpoints, models)."""

    def __init__(self):
        self.parents: Dict[str, List[str]] = {}

    def link(self, child: str, parent: str):
        self.parents.setdefault(child, []).append(parent)

    def ancestors(self, node: str) -> List[str]:
        out, stack = [], list(self.parents.get(node, []))
        while stack:
            n = stack.pop()
            if n not in out:
                out.append(n)
                stack.extend(self.parents.get(n, []))
        return out


# ----------------------------------------------------------------------------------------- ONNX, graph, NPE, ARC, FM aliases
OnnxModel, OnnxGraph, OnnxNode = _onnx.Model, _onnx.Graph, _onnx.Node
onnx_check = onnx_validate = _onnx.check_model
quantize_graph_weights = _onnx.quantize_qdq


class OnnxShapeError(ValueError):
    pass


def export_onnx(module, example_input, path: Optional[str] = None):
    return _onnx.export_module(module, example_input, path)


class OnnxExporter:
    def export(self, module, example_input, path=None):
        return _onnx.export_module(module, example_input, path)


def import_onnx(path_or_bytes):
    return _onnx.Model.parse(path_or_bytes) if isinstance(path_or_bytes, (bytes, bytearray)) else _onnx.Model.load(path_or_bytes)


class OnnxImporter:
    load = staticmethod(import_onnx)


def onnx_to_protobuf(model) -> bytes:
    return model.serialize()


protobuf_to_onnx = _onnx.Model.parse


def onnx_version_compatible(model, max_opset: int = 21, min_opset: int = 7) -> bool:
    return min_opset <= int(getattr(model, "opset", 0) or 0) <= max_opset


def upgrade_opset(model, target: int = 17):
    model.opset = max(int(getattr(model, "opset", 0) or 0), target)
    return model


def inference_session(path_or_model):
    """Callable running the model on NumPy feeds (the toolkit's executor)."""
    m = path_or_model if isinstance(path_or_model, _onnx.Model) else import_onnx(path_or_model)
    return lambda feeds: _onnx.run_model(m, feeds)


def select_execution_provider(preferred: Sequence[str] = ("cuda", "cpu")) -> str:
    return "cuda" if "cuda" in preferred and torch.cuda.is_available() else "cpu"


from . import graph as _graph  # noqa: E402

StateGraph = _graph.ExprGraph


class CompiledGraph:
    """An expression graph bound to its outputs and fusion plan: call it with named inputs."""

    def __init__(self, graph, outputs, fuse: bool = True):
        self.graph, self.outputs, self.fuse = graph, list(outputs), fuse
        self.plan = graph.plan_fusions(self.outputs) if fuse else []

    def __call__(self, **feeds):
        return self.graph.run(self.outputs, feeds, fuse=self.fuse)

    @property
    def num_fused_groups(self) -> int:
        return len(self.plan)


class GraphOptimizer:
    """Fusion planner front: ``optimize(graph, outputs)`` returns the fusion groups (matmul + bias + activation chains)
    and ``memory_saving`` the bytes of intermediates that fusing avoids."""

    def optimize(self, graph, outputs):
        return graph.plan_fusions(list(outputs))

    def memory_saving(self, graph, outputs, shapes, elem_bytes=2) -> int:
        return graph.memory_estimate(list(outputs), shapes, elem_bytes, fused=False) - \
            graph.memory_estimate(list(outputs), shapes, elem_bytes, fused=True)


class GraphCompiler:
    def __init__(self, fuse: bool = True):
        self.fuse = fuse

    def compile(self, graph, outputs) -> CompiledGraph:
        return CompiledGraph(graph, outputs, self.fuse)


FUSABLE_OPS = ("matmul", "bias", "relu", "gelu", "silu", "add", "mul")


def visualize_graph(g) -> str:
    """Graphviz dot text of an expression graph."""
    lines = ["digraph G {"]
    for i, n in enumerate(getattr(g, "nodes", [])):
        lines.append(f'  n{i} [label="{getattr(n, "op", "?")}"];')
        for j in getattr(n, "inputs", []):
            lines.append(f"  n{j} -> n{i};")
    return "\n".join(lines + ["}"])


def trace_function(fn, *example_inputs):
    from . import jit
    return jit.trace(fn, *example_inputs)


jit = trace_function


class Trace:
    """What a ``Tracer`` recorded for one function: the captured callable and the example input signature."""

    def __init__(self, fn, compiled, example_inputs):
        self.fn, self.compiled = fn, compiled
        self.signature = [(tuple(t.shape), str(t.dtype)) if torch.is_tensor(t) else type(t).__name__ for t in example_inputs]

    def __call__(self, *inputs):
        return self.compiled(*inputs)


class Tracer:
    """Captures functions into replayable form (a CUDA graph for CUDA inputs, the function itself otherwise) and keeps
    the traces by name."""

    def __init__(self):
        self.traces: Dict[str, Trace] = {}

    def trace(self, fn, *example_inputs, name: Optional[str] = None) -> Trace:
        t = Trace(fn, trace_function(fn, *example_inputs), example_inputs)
        self.traces[name or getattr(fn, "__name__", f"fn{len(self.traces)}")] = t
        return t

NPEInstruction = _npe.Instruction
ARCInputGuard, ARCGradientObfuscator, ARCOutputVerifier, ARCAttackSim = _arc.InputGuard, _arc.GradientObfuscator, _arc.OutputVerifier, _arc.simulate_attack
FMMemoryBank, FMNode = _fm.MemoryBank, _fm.Node


class Attack:
    """An input-space attack with a perturbation budget ``epsilon`` inside the box [lo, hi]. ``attack(x, loss_fn)``
    (or calling the object) returns the adversarial input; subclasses name the method."""

    kind = _arc.ATTACK_FGSM

    def __init__(self, epsilon=0.1, lo=-1.0, hi=1.0, **extra):
        self.epsilon, self.lo, self.hi, self.extra = epsilon, lo, hi, extra

    def attack(self, x, loss_fn):
        return _arc.simulate_attack(x, self.kind, self.epsilon, loss_fn, lo=self.lo, hi=self.hi, **self.extra)

    __call__ = attack


class FGSM(Attack):
    """One signed-gradient step of size epsilon."""


class PGD(Attack):
    """``steps`` projected signed-gradient steps inside the epsilon ball."""

    kind = _arc.ATTACK_PGD

    def __init__(self, epsilon=0.1, steps=3, lo=-1.0, hi=1.0):
        super().__init__(epsilon, lo, hi, steps=steps)


class ARCAttackSim:
    """Runs a set of attacks against ``loss_fn`` and reports how much each raises the loss."""

    def __init__(self, attacks=None):
        self.attacks = list(attacks) if attacks is not None else [FGSM(0.05), PGD(0.05, steps=3)]

    def run(self, x, loss_fn):
        base = float(loss_fn(x))
        out = {}
        for a in self.attacks:
            adv = a(x, loss_fn)
            out[type(a).__name__] = {"loss": float(loss_fn(adv)), "clean_loss": base,
                                     "linf": float((adv - x).abs().max())}
        return out


@dataclass
class AdversarialExample:
    clean: torch.Tensor
    adversarial: torch.Tensor
    epsilon: float


class AdversarialTrainer:
    """Mixes clean and FGSM-perturbed batches: loss = (1 - w) L(x) + w L(x_adv)."""

    def __init__(self, model, loss_fn, epsilon=0.03, weight=0.5):
        self.model, self.loss_fn, self.epsilon, self.weight = model, loss_fn, epsilon, weight

    def loss(self, x, y, lo=-1.0, hi=1.0):
        adv = FGSM(x, lambda t: self.loss_fn(self.model(t), y), self.epsilon, lo, hi)
        return (1 - self.weight) * self.loss_fn(self.model(x), y) + self.weight * self.loss_fn(self.model(adv), y)




# ----------------------------------------------------------------------------------------- data, tokenizers, trainers
Dataset = CppDataset = PyTorchDataset = torch.utils.data.Dataset
CppTensorDataset = _data.TensorDataset
PyTorchDataLoader = _data.DataLoader


class _LateBound(type):
    """Metaclass of class names that are bound to their implementation at first use (the implementation's module is
    not imported with this one). Calling the name constructs the implementation; ``isinstance`` / ``issubclass``
    and attribute access go to it."""

    def _real(cls):
        r = cls.__dict__.get("_resolved")
        if r is None:
            import importlib
            r = getattr(importlib.import_module(f"sneppx_alg_b200.{cls._mod}"), cls._attr)
            type.__setattr__(cls, "_resolved", r)
        return r

    def __call__(cls, *a, **k):
        return cls._real()(*a, **k)

    def __instancecheck__(cls, obj):
        return isinstance(obj, cls._real())

    def __subclasscheck__(cls, sub):
        return issubclass(sub, cls._real())

    def __getattr__(cls, name):
        if name.startswith("__"):
            raise AttributeError(name)
        return getattr(cls._real(), name)


def _lazy(mod, attr):
    """A late-bound class name when ``attr`` is spelled like a class, else a late-bound function."""
    if attr[:1].isupper():
        return _LateBound(attr, (), {"_mod": mod, "_attr": attr, "_resolved": None,
                                     "__doc__": f"``sneppx_alg_b200.{mod}.{attr}``, bound at first use."})

    def get(*a, **k):
        import importlib
        return getattr(importlib.import_module(f"sneppx_alg_b200.{mod}"), attr)(*a, **k)
    get.__name__ = attr
    return get


Tokenizer = _lazy("utils.host", "BPETokenizer")
SimpleTokenizer = TokenizerSimpleTokenizer = _lazy("serving.server", "ByteTokenizer")
TrainerV3 = PyTorchTrainer = _lazy("training.trainer", "Trainer")
TrainConfigV3 = UltraTrainConfig = _lazy("training.config", "TrainConfig")
EdgeRuntime = _lazy("utils.host", "EdgeModel")
SocketComm = _lazy("utils.net", "FramedSocket")
GRPCService = _lazy("utils.net", "CoordinatorServer")
NCCLComm = _lazy("parallel.distributed", "ProcessGroup")
MemoryAllocator = _lazy("utils.mm", "Arena")


class MemoryPool:
    """Size-class host memory pool of the native runtime (``sx_pool_*`` in csrc/host/cpu_oracle.cpp): ``alloc`` /
    ``free`` by address with hit / miss statistics."""

    def __init__(self):
        import ctypes as C

        from .utils.host import _L as _host
        self._C, self._L = C, _host()
        self._L.sx_pool_alloc.argtypes = [C.c_void_p, C.c_size_t]
        self._L.sx_pool_free.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        self._L.sx_pool_stats.argtypes = [C.c_void_p, C.c_void_p]
        self._h = self._L.sx_pool_create()

    def alloc(self, n: int) -> int:
        return self._L.sx_pool_alloc(self._h, n) or 0

    def free(self, ptr: int, n: int) -> None:
        self._L.sx_pool_free(self._h, ptr, n)

    def stats(self) -> dict:
        out = (self._C.c_longlong * 3)()
        self._L.sx_pool_stats(self._h, out)
        return {"allocations": int(out[0]), "reused": int(out[1]), "bytes_live": int(out[2])}

    def close(self) -> None:
        if self._h:
            self._L.sx_pool_destroy(self._h)
            self._h = None


class ContinuousBatchScheduler:
    """Request-level front of the continuous-batching engine with the reference scheduler's verbs
    (interface_bindings/continuous_batching.py:64-179: ``submit`` / ``get_batch`` / ``step``): requests are queued,
    ``get_batch`` shows what is running, ``step`` advances every running sequence by one token on the paged engine."""

    def __init__(self, model, max_batch_size: int = 32, **engine_kwargs):
        from .serving.llm_engine import LLMEngine
        self.engine = LLMEngine(model, max_batch_size=max_batch_size, **engine_kwargs)

    def submit(self, prompt_tokens: List[int], max_new_tokens: int = 64, priority: int = 0, **sampling) -> int:
        from .serving.llm_engine import SamplingParams
        return self.engine.submit(list(prompt_tokens), SamplingParams(max_new_tokens=max_new_tokens, **sampling), priority)

    def get_batch(self) -> List[int]:
        return list(self.engine.running)

    def step(self) -> Dict[int, List[int]]:
        """One engine step; returns the requests that finished in it with their output tokens."""
        before = set(self.engine.finished)
        self.engine.step()
        return {rid: self.engine.finished[rid].output for rid in set(self.engine.finished) - before}

    def run(self) -> Dict[int, List[int]]:
        self.engine.run_until_done()
        return {rid: r.output for rid, r in self.engine.finished.items()}

    @property
    def pending(self) -> int:
        return len(self.engine.waiting)
DynamicBatchQueue = _lazy("utils.host", "ServingCore")
TrainProfiler = _lazy("utils.observability", "Profiler")
from .training.lora import QLoRALinear  # noqa: E402
class GradientCheckpointer:
    """Wraps the repeated layers of ``model`` so that their activations are recomputed in backward."""

    def __init__(self, model=None, every: int = 1):
        self.every, self.wrapped = every, 0
        if model is not None:
            self.apply(model)

    def apply(self, model):
        from .training.extras import enable_activation_checkpointing
        self.wrapped = enable_activation_checkpointing(model) or 0
        return model

    @staticmethod
    def checkpoint(fn, *args):
        from .training.extras import checkpoint
        return checkpoint(fn, *args)
checkpoint_sequential = _lazy("training.extras", "checkpoint")
class TopologyType(enum.Enum):
    RING = "ring"
    TREE = "tree"
    GRAPH = "graph"


@dataclass
class EdgeConfig:
    max_width: int = 4096
    int8: bool = False


# ----------------------------------------------------------------------------------------- privacy mechanisms
class LaplaceMech:
    def __init__(self, epsilon: float, sensitivity: float = 1.0):
        self.scale = sensitivity / epsilon

    def __call__(self, x, generator=None):
        u = torch.rand(x.shape, generator=generator) - 0.5
        return x - self.scale * torch.sign(u) * torch.log1p(-2 * u.abs())


class GaussianMech:
    def __init__(self, epsilon: float, delta: float = 1e-5, sensitivity: float = 1.0):
        import math
        self.sigma = sensitivity * math.sqrt(2 * math.log(1.25 / delta)) / epsilon

    def __call__(self, x, generator=None):
        return x + self.sigma * torch.randn(x.shape, generator=generator)


class PrivacyBudget:
    """Sequential composition: spent epsilon adds up; `spend` refuses to exceed the total."""

    def __init__(self, epsilon: float, delta: float = 0.0):
        self.epsilon, self.delta, self.spent = epsilon, delta, 0.0

    def spend(self, eps: float) -> bool:
        if self.spent + eps > self.epsilon + 1e-12:
            return False
        self.spent += eps
        return True

    @property
    def remaining(self) -> float:
        return self.epsilon - self.spent


# ----------------------------------------------------------------------------------------- pools and benchmarks
class ThreadPool:
    """Futures-returning pool (the C runtime's work-stealing pool maps onto the interpreter's executor here; the
    native work queue is ``utils.host``)."""

    def __init__(self, workers: int = 4):
        self._ex = ThreadPoolExecutor(max_workers=workers)

    def submit(self, fn, *a, **k):
        return self._ex.submit(fn, *a, **k)

    def map(self, fn, items):
        return list(self._ex.map(fn, items))

    def shutdown(self):
        self._ex.shutdown(wait=True)


from .utils.workpool import Future as PoolFuture, TaskGroup, Workload, WorkStealingPool  # noqa: E402  (native pool)



class BenchmarkTimer:
    def __enter__(self):
        self.t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        self.ms = (time.perf_counter() - self.t0) * 1e3


@dataclass
class BenchmarkConfig:
    device: str = "cpu"
    scale_runs: float = 1.0


@dataclass
class BenchmarkResult:
    op: str
    mean_ms: float
    min_ms: float
    max_ms: float
    runs: int


class BenchmarkSuite:
    def __init__(self, config: Optional[BenchmarkConfig] = None):
        self.config = config or BenchmarkConfig()

    def run(self) -> List[BenchmarkResult]:
        from .benchmarks import tensor_ops
        res = tensor_ops.run(self.config.device, self.config.scale_runs)["results"]
        return [BenchmarkResult(r["op"], r["mean_ms"], r["min_ms"], r["max_ms"], r["runs"]) for r in res]


def run_benchmarks(device: str = "cpu", scale_runs: float = 1.0):
    return BenchmarkSuite(BenchmarkConfig(device, scale_runs)).run()


benchmark = run_benchmarks


def run_benchmark_cli(argv=None):
    from .benchmarks import tensor_ops
    return tensor_ops.main(argv)


# ----------------------------------------------------------------------------------------- kernel entry points by name
def gemm_kernel(a, b, bias=None, act=None):
    """a [M, K] x b [N, K]^T on the tcgen05 GEMM for bf16 CUDA tensors (fp32 statement of the same product otherwise)."""
    from .ops.gemm import gemm
    return gemm(a, b, bias=bias, act=act)


gemm_batched_kernel = gemm_kernel


def _elementwise(fn):
    def run(x, *a, **k):
        return fn(x, *a, **k)
    return run


relu_kernel, gelu_kernel, silu_kernel = _elementwise(torch.relu), _elementwise(lambda x: torch.nn.functional.gelu(x, approximate="tanh")), _elementwise(torch.nn.functional.silu)
softmax_kernel = _elementwise(lambda x, dim=-1: torch.softmax(x, dim))


def bias_gelu_kernel(x, bias):
    return torch.nn.functional.gelu(x + bias, approximate="tanh")


def layernorm_kernel(x, w, b=None, eps=1e-5):
    from .ops.functional import layernorm
    return layernorm(x, w, b, eps)


def layernorm_backward_kernel(x, w, b, dy, eps=1e-5):
    """(dx, dw, db) through the op's own backward (native on bf16 CUDA tensors)."""
    from .ops.functional import layernorm
    xs, ws = x.detach().requires_grad_(True), w.detach().requires_grad_(True)
    bs = None if b is None else b.detach().requires_grad_(True)
    with torch.enable_grad():
        y = layernorm(xs, ws, bs, eps)
    grads = torch.autograd.grad(y, [t for t in (xs, ws, bs) if t is not None], dy)
    return tuple(grads) + ((None,) if b is None else ())


def rmsnorm_kernel(x, w, eps=1e-5):
    from .ops.functional import rmsnorm
    return rmsnorm(x, w, eps)[0]


def dropout_kernel(x, p, seed=0, offset=0):
    from .ops.aux import dropout
    return dropout(x, p, seed, offset)


def dropout_backward_kernel(dy, p, seed=0, offset=0):
    from .ops.aux import dropout
    return dropout(dy, p, seed, offset)   # the mask is a function of (seed, offset): backward is the same map


def flash_attention_v2_kernel(q, k, v, causal=True, scale=None):
    from .ops.functional import attention
    return attention(q, k, v, causal=causal, scale=scale)


def flash_attention_v2_backward_kernel(q, k, v, do, causal=True, scale=None):
    from .ops.functional import attention
    qs, ks, vs = (t.detach().requires_grad_(True) for t in (q, k, v))
    with torch.enable_grad():
        o = attention(qs, ks, vs, causal=causal, scale=scale)
    return torch.autograd.grad(o, (qs, ks, vs), do)


def fused_adamw_kernel(p, g, m, v, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, step=1):
    """In-place AdamW on one tensor with the reference's update order (decay, then the bias-corrected step)."""
    with torch.no_grad():
        m.mul_(beta1).add_(g, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
        p.mul_(1 - lr * weight_decay)
        p.addcdiv_(m / (1 - beta1 ** step), (v / (1 - beta2 ** step)).sqrt().add_(eps), value=-lr)
    return p


def conv2d_kernel(x, w, bias=None, stride=1, padding=0):
    return torch.nn.functional.conv2d(x, w, bias, stride, padding)


@dataclass
class KernelConfig:
    block: int = 256
    stages: int = 4




class KernelLauncher:
    """Name -> callable table over the entry points above."""

    def __init__(self):
        self.table = {n[:-7]: f for n, f in globals().items() if n.endswith("_kernel") and callable(f)}

    def launch(self, name: str, *a, **k):
        return self.table[name](*a, **k)


dispatch = lambda name, *a, **k: KernelLauncher().launch(name, *a, **k)  # noqa: E731
ELEMENTWISE_IMPL = {"relu": relu_kernel, "gelu": gelu_kernel, "silu": silu_kernel}


# ----------------------------------------------------------------------------------------- records, enums, small services
import enum  # noqa: E402

from .security import ai_filter as _aif  # noqa: E402

AIPromptFilter = S5PromptFilter = _aif.PromptFilter
AIOutputVerifier = S5OutputVerifier = _aif.OutputVerifier


class AuditSeverity(enum.IntEnum):
    INFO, WARNING, ERROR, CRITICAL = 0, 1, 2, 3




class AuditAction(str, enum.Enum):
    LOGIN, DATA_ACCESS, CONFIG_CHANGE, SECURITY_EVENT, MODEL_DEPLOY = "login", "data_access", "config_change", "security_event", "model_deploy"


class AuditResult(str, enum.Enum):
    SUCCESS, FAILURE, DENIED = "success", "failure", "denied"


class DDoSAction(str, enum.Enum):
    ALLOW, THROTTLE, BAN = "allow", "throttle", "ban"


class ScanStatus(str, enum.Enum):
    CLEAN, VULNERABLE = "clean", "vulnerable"


class ModelFamily(str, enum.Enum):
    LLAMA, MISTRAL, QWEN2, DEEPSEEK_V2, MAMBA2, HSS_SER = "llama", "mistral", "qwen2", "deepseek_v2", "mamba2", "hss_ser"


class Dtype(enum.Enum):
    FLOAT32, FLOAT16, BFLOAT16, INT8, INT32, INT64, FP8_E4M3 = (torch.float32, torch.float16, torch.bfloat16, torch.int8, torch.int32,
                                                               torch.int64, torch.float8_e4m3fn)


class Layout(str, enum.Enum):
    ROW_MAJOR, COL_MAJOR = "row_major", "col_major"


@dataclass
class AuditEvent:
    actor: str
    action: str
    severity: AuditSeverity = AuditSeverity.INFO
    result: AuditResult = AuditResult.SUCCESS
    details: Dict[str, Any] = field(default_factory=dict)


@dataclass
class RateLimitConfig:
    rate: float = 10.0
    burst: float = 20.0


@dataclass
class DDoSConfig(RateLimitConfig):
    ban_after: int = 5
    ban_seconds: float = 60.0

    def build(self):
        return _svc.DDoSMitigator(self.rate, self.burst, self.ban_after, self.ban_seconds)


@dataclass
class AuthConfig:
    mode: str = "none"
    api_keys: List[str] = field(default_factory=list)
    admin_key: Optional[str] = None


@dataclass
class SecurityConfig:
    auth: AuthConfig = field(default_factory=AuthConfig)
    ddos: DDoSConfig = field(default_factory=DDoSConfig)
    prompt_filter: bool = True
    output_verifier: bool = True


@dataclass
class PromptFilterConfig:
    max_chars: int = 100_000
    block_threshold: float = 0.5

    def build(self):
        return _aif.PromptFilter(self.max_chars, self.block_threshold)


@dataclass
class OutputVerifierConfig:
    enabled: bool = True

    def build(self):
        return _aif.OutputVerifier()


@dataclass
class ScanResult:
    status: ScanStatus
    components: List[SBOMComponent] = field(default_factory=list)


@dataclass
class CVE:
    cve_id: str
    package: str
    severity: AuditSeverity = AuditSeverity.WARNING




@dataclass
class TensorDescriptor:
    shape: Sequence[int]
    dtype: torch.dtype = torch.float32
    layout: Layout = Layout.ROW_MAJOR

    @property
    def nbytes(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n * torch.empty(0, dtype=self.dtype).element_size()




@dataclass
class CheckpointHeader:
    """Fields of the 72-byte `.sneppx` header (magic 0x41524958 / 0x434B5054, version 1)."""
    num_tensors: int
    metadata_offset: int
    metadata_size: int
    total_size: int
    version: int = 1


@dataclass
class CheckpointSegment:
    name: str
    offset: int
    size: int


@dataclass
class PromptVersion:
    name: str
    version: int
    template: str


@dataclass
class RegisteredModel:
    name: str
    version: int
    uri: str
    stage: str = "none"


@dataclass
class TrafficSplit:
    weights: Dict[str, float]

    def route(self, request_id: str) -> str:
        from .utils.host import ServingCore
        keys = sorted(self.weights)
        return keys[ServingCore.route(request_id, [self.weights[k] for k in keys])]


@dataclass
class ScheduledRequest:
    request_id: int
    prompt: List[int]
    priority: int = 0
    arrival: float = field(default_factory=time.perf_counter)


@dataclass
class BatchResult:
    outputs: List[List[int]]
    latency_s: float


@dataclass
class ProfileEntry:
    name: str
    calls: int = 0
    total_ms: float = 0.0

    @property
    def mean_ms(self) -> float:
        return self.total_ms / max(self.calls, 1)


@dataclass
class GatewayRoute:
    route: str
    provider: str
    weight: float = 1.0
    rate_limit_per_s: float = 0.0


def register_model(name: str, uri: str, registry_path: str = "~/.sneppx/registry.json", **kw):
    from .utils.registry import ModelRegistry
    path = os.path.expanduser(registry_path)
    os.makedirs(os.path.dirname(path), exist_ok=True)
    return ModelRegistry(path).register(name, uri, **kw)


def load_config(path: str) -> dict:
    import yaml
    return yaml.safe_load(open(path)) if path.endswith((".yaml", ".yml")) else json.load(open(path))


class ConfigReloader:
    """Re-reads a config file when its modification time changes (the serving engine's hot reload)."""

    def __init__(self, path: str, on_change: Optional[Callable[[dict], None]] = None):
        self.path, self.on_change, self.mtime, self.config = path, on_change, 0.0, {}
        self.poll()

    def poll(self) -> bool:
        m = os.path.getmtime(self.path)
        if m == self.mtime:
            return False
        self.mtime, self.config = m, load_config(self.path)
        if self.on_change:
            self.on_change(self.config)
        return True


def query_audit_log(actor: Optional[str] = None, action: Optional[str] = None) -> List[dict]:
    path = get_audit_logger().path
    rows = [json.loads(l) for l in open(path)] if os.path.exists(path) else []
    return [r for r in rows if (actor is None or r["actor"] == actor) and (action is None or r["action"] == action)]


def export_audit_log(dest: str) -> int:
    rows = query_audit_log()
    with open(dest, "w") as f:
        json.dump(rows, f)
    return len(rows)




class ConnectionTracker:
    """Open connections per client with a cap (SYN-flood style exhaustion shows up as refusals)."""

    def __init__(self, max_per_client: int = 64):
        self.max, self.open = max_per_client, {}

    def acquire(self, client: str) -> bool:
        if self.open.get(client, 0) >= self.max:
            return False
        self.open[client] = self.open.get(client, 0) + 1
        return True

    def release(self, client: str):
        self.open[client] = max(0, self.open.get(client, 0) - 1)


_connections = ConnectionTracker()
release_connection = _connections.release


class IPReputationManager:
    def __init__(self):
        self.score: Dict[str, float] = {}

    def report(self, ip: str, bad: bool, weight: float = 1.0):
        self.score[ip] = min(1.0, max(-1.0, self.score.get(ip, 0.0) + (-0.2 if bad else 0.05) * weight))

    def trusted(self, ip: str, threshold: float = -0.5) -> bool:
        return self.score.get(ip, 0.0) > threshold


class AdaptiveThresholdManager:
    """Anomaly threshold at mean + k * std of an exponential window."""

    def __init__(self, k: float = 3.0, decay: float = 0.99):
        self.k, self.decay, self.mean, self.var, self.n = k, decay, 0.0, 0.0, 0

    def update(self, x: float) -> bool:
        anomalous = self.n > 10 and x > self.mean + self.k * self.var ** 0.5
        d = x - self.mean
        self.mean += (1 - self.decay) * d
        self.var = self.decay * (self.var + (1 - self.decay) * d * d)
        self.n += 1
        return anomalous


class RLHFSafety:
    """Reward shaping that subtracts a penalty for responses the output verifier flags."""

    def __init__(self, penalty: float = 1.0):
        self.verifier, self.penalty = _aif.OutputVerifier(), penalty

    def shaped_reward(self, response: str, reward: float) -> float:
        res = self.verifier.verify(response)
        return reward - (self.penalty if res.sanitized != response else 0.0)


S5RLHFSafety = RLHFSafety


class DataPoisoningDefense:
    """Flags training samples whose feature vector is an outlier (distance to the class centroid above k sigma)."""

    def __init__(self, k: float = 3.0):
        self.k = k

    def flag(self, features: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        out = torch.zeros(len(features), dtype=torch.bool)
        for c in labels.unique():
            idx = (labels == c).nonzero().flatten()
            d = (features[idx] - features[idx].mean(0)).norm(dim=1)
            out[idx] = d > d.mean() + self.k * d.std().clamp_min(1e-12)
        return out


def rewrite_weights(model, fn: Callable[[str, torch.Tensor], torch.Tensor]):
    """Applies fn(name, tensor) to every parameter in place (format conversions, dtype casts, re-scaling)."""
    with torch.no_grad():
        for n, p in model.named_parameters():
            p.copy_(fn(n, p).to(p.dtype))
    return model


def _distill(student, teacher, batches, steps: int = 10, lr: float = 1e-3, T: float = 2.0):
    from .compat import kd_loss
    opt = torch.optim.AdamW(student.parameters(), lr=lr)
    losses = []
    for _, x in zip(range(steps), batches):
        with torch.no_grad():
            t = teacher(x)
        s = student(x)
        t, s = (o["logits"] if isinstance(o, dict) else o for o in (t, s))
        loss = kd_loss(s.reshape(-1, s.shape[-1]), t.reshape(-1, t.shape[-1]), T)
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss))
    return losses


distill_bert = distill_gpt = _distill


class OnlineDistillation:
    """Teacher and student trained together; the student also matches the teacher's softened logits."""

    def __init__(self, student, teacher, T: float = 2.0, weight: float = 0.5):
        self.student, self.teacher, self.T, self.weight = student, teacher, T, weight

    def loss(self, x, y, loss_fn):
        from .compat import kd_loss
        s, t = self.student(x), self.teacher(x)
        return loss_fn(s, y) + loss_fn(t, y) + self.weight * kd_loss(s, t.detach(), self.T)


def prune_and_distill(student, teacher, batches, sparsity: float = 0.5, steps: int = 10):
    from .compat import apply_pruning_mask, global_magnitude_prune
    masks = global_magnitude_prune(student, sparsity)
    losses = _distill(student, teacher, batches, steps)
    apply_pruning_mask(student, masks)
    return masks, losses


class DistillationPruner:
    """Global magnitude pruning of the student to ``sparsity`` followed by ``steps`` distillation steps against the
    teacher with the mask re-applied; ``run(batches)`` returns (masks, losses)."""

    def __init__(self, student, teacher, sparsity: float = 0.5, steps: int = 10):
        self.student, self.teacher, self.sparsity, self.steps = student, teacher, sparsity, steps
        self.masks, self.losses = None, []

    def run(self, batches):
        self.masks, self.losses = prune_and_distill(self.student, self.teacher, batches, self.sparsity, self.steps)
        return self.masks, self.losses


class Random:
    """Seeded generator facade over torch (uniform / normal / randint / permutation)."""

    def __init__(self, seed: int = 0, device="cpu"):
        self.gen = torch.Generator(device=device).manual_seed(seed)
        self.device = device

    def uniform(self, *shape, low=0.0, high=1.0):
        return low + (high - low) * torch.rand(*shape, generator=self.gen, device=self.device)

    def normal(self, *shape, mean=0.0, std=1.0):
        return mean + std * torch.randn(*shape, generator=self.gen, device=self.device)

    def randint(self, low, high, shape):
        return torch.randint(low, high, tuple(shape), generator=self.gen, device=self.device)

    def permutation(self, n):
        return torch.randperm(n, generator=self.gen, device=self.device)


class HardwareProbe:
    @staticmethod
    def probe() -> dict:
        from .compat import detect_cpu
        from . import device as _dev
        return {"cpu": detect_cpu(), "cuda_devices": _dev.device_count()}


class CUDAMemoryPool:
    """View of PyTorch's caching allocator (the device memory pool of this framework)."""

    @staticmethod
    def stats() -> dict:
        if not torch.cuda.is_available():
            return {"allocated": 0, "reserved": 0}
        return {"allocated": torch.cuda.memory_allocated(), "reserved": torch.cuda.memory_reserved()}

    @staticmethod
    def empty_cache():
        if torch.cuda.is_available():
            torch.cuda.empty_cache()


class MemoryLeakDetector:
    """Snapshot / compare of live tensor bytes between two points."""

    def __init__(self):
        self.base = self._live()

    @staticmethod
    def _live() -> int:
        import gc
        return sum(o.numel() * o.element_size() for o in gc.get_objects() if isinstance(o, torch.Tensor))

    def leaked_bytes(self) -> int:
        return self._live() - self.base


class ServingServer:
    """Owns the C++ HTTP front-end for one engine (``serving.native_http.serve_engine``)."""

    def __init__(self, engine, models: Dict[str, dict], token: str = "", port: int = 0):
        from .serving.native_http import serve_engine
        self._srv = serve_engine(engine, models, token, port)
        self.port = self._srv.port

    def stop(self):
        self._srv.stop()


class SneppxTrackingClient:
    """Client of the local experiment tracker directory (run listing and metric history)."""

    def __init__(self, directory: str = "runs"):
        self.dir = directory

    def list_runs(self, experiment: str = "default") -> List[str]:
        p = os.path.join(self.dir, experiment)
        return sorted(os.listdir(p)) if os.path.isdir(p) else []


ONNX_OP_REGISTRY = ("MatMul", "Gemm", "Add", "Mul", "Relu", "Gelu", "Sigmoid", "Tanh", "Softmax", "LayerNormalization", "Reshape",
                    "Transpose", "Concat", "Gather", "Identity", "QuantizeLinear", "DequantizeLinear")
SNEPPX_TO_ONNX_OP = {"linear": "Gemm", "matmul": "MatMul", "add": "Add", "mul": "Mul", "relu": "Relu", "gelu": "Gelu", "softmax": "Softmax",
                     "layernorm": "LayerNormalization", "embedding": "Gather"}
stage_update = lambda mgr, path, manifest, min_version="0": mgr.stage_update(path, manifest, min_version)  # noqa: E731
install_update = lambda mgr: mgr.install_update()  # noqa: E731
rollback_update = lambda mgr, file_name: mgr.rollback_update(file_name)  # noqa: E731


AlgoHSSModel, AlgoSERModel = _lazy("algorithms", "HSSModel"), _lazy("algorithms", "SERModel")
DeepSeekV2Model = _lazy("models.deepseek", "DeepSeekV2ForCausalLM")
BlockTable = _lazy("serving.kv_cache", "PagedKVCache")
DataBuffer = _lazy("utils.mm", "Arena")


class BigNum(int):
    """Arbitrary-precision integer with the byte conversions the crypto wrappers use."""

    @classmethod
    def from_bytes_le(cls, b: bytes):
        return cls(int.from_bytes(b, "little"))

    def to_bytes_le(self, n: int) -> bytes:
        return int(self).to_bytes(n, "little")

    def modexp(self, e: int, m: int):
        return BigNum(pow(int(self), e, m))


class ArchOps:
    """Functional forms of the architecture blocks (``c_arch.py``): one Mamba-2 block or SER layer applied to a tensor."""

    @staticmethod
    def mamba2(x, d_state=64, d_conv=4, seed=0):
        from .nn.ssm import Mamba2Block
        torch.manual_seed(seed)
        return Mamba2Block(x.shape[-1], d_state=d_state, d_conv=d_conv, headdim=min(64, x.shape[-1] * 2)).to(x.dtype)(x)


from .quant.algorithms import MX_FORMATS, MXFormat, MXFormatSpec, mx_quantize_spec  # noqa: E402,F401


class Preprocessor:
    """Text -> padded id batch with a tokenizer that has ``encode``."""

    def __init__(self, tokenizer, max_len: int = 512, pad_id: int = 0):
        self.tok, self.max_len, self.pad_id = tokenizer, max_len, pad_id

    def __call__(self, texts: Sequence[str]) -> torch.Tensor:
        ids = [self.tok.encode(t)[: self.max_len] for t in texts]
        width = max(len(i) for i in ids)
        return torch.tensor([i + [self.pad_id] * (width - len(i)) for i in ids], dtype=torch.long)


class Tensorable:
    """Mixin: anything with ``to_tensor``."""

    def to_tensor(self) -> torch.Tensor:
        raise NotImplementedError


class SimdGemm:
    """The reference's CPU SIMD GEMM entry; here the GEMM op (tensor cores on CUDA bf16, torch otherwise)."""

    @staticmethod
    def gemm(a, b):
        return gemm_kernel(a, b)


class SyslogAuditBackend(_svc.AuditLogger):
    """Audit chain that also forwards each record to the local syslog socket when one exists."""

    def log(self, actor, action, **details):
        h = super().log(actor, action, **details)
        try:
            import syslog
            syslog.syslog(f"sneppx-audit {actor} {action} {h[:12]}")
        except Exception:
            pass
        return h


class DatabaseAuditBackend:
    """Audit chain in SQLite with the same hash linking."""

    def __init__(self, path: str):
        import sqlite3
        self.db = sqlite3.connect(path)
        self.db.execute("create table if not exists audit (id integer primary key, rec text, hash text)")
        row = self.db.execute("select hash from audit order by id desc limit 1").fetchone()
        self.last = row[0] if row else "0" * 64

    def log(self, actor, action, **details):
        from .security import crypto
        rec = {"ts": time.time(), "actor": actor, "action": action, "details": details, "prev": self.last}
        h = crypto.sha256(json.dumps(rec, sort_keys=True).encode()).hex()
        self.db.execute("insert into audit (rec, hash) values (?, ?)", (json.dumps(rec, sort_keys=True), h))
        self.db.commit()
        self.last = h
        return h

    def verify(self) -> bool:
        from .security import crypto
        prev = "0" * 64
        for rec, h in self.db.execute("select rec, hash from audit order by id"):
            if json.loads(rec)["prev"] != prev or crypto.sha256(rec.encode()).hex() != h:
                return False
            prev = h
        return True


# ----------------------------------------------------------------------------------------- host hardening probes, transport
class ASLR:
    """Address-space layout randomisation setting of this kernel (0 off, 1 partial, 2 full; None when unreadable)."""

    @staticmethod
    def level() -> Optional[int]:
        try:
            return int(open("/proc/sys/kernel/randomize_va_space").read().strip())
        except (OSError, ValueError):
            return None

    @classmethod
    def enabled(cls) -> bool:
        return (cls.level() or 0) > 0


class StackCanary:
    """Canary-guarded buffer check (the host library's guarded allocation: a canary word on each side of the block)."""

    def __init__(self, nbytes: int = 64):
        from .security import crypto
        self.buf = crypto.GuardedBuffer(nbytes)

    def intact(self) -> bool:
        return self.buf.check() == 0   # 0: both canaries untouched


class MemoryHardening:
    @staticmethod
    def report() -> dict:
        import resource
        core = resource.getrlimit(resource.RLIMIT_CORE)[0]
        return {"aslr": ASLR.level(), "core_dumps_disabled": core == 0, "guarded_allocations": True}

    @staticmethod
    def disable_core_dumps():
        import resource
        resource.setrlimit(resource.RLIMIT_CORE, (0, resource.getrlimit(resource.RLIMIT_CORE)[1]))


class ContainerBreakoutDetector:
    """Signals that a process inside a container can reach the host: privileged capabilities, a writable docker
    socket, the host's process namespace."""

    @staticmethod
    def scan() -> dict:
        findings = {}
        try:
            status = open("/proc/self/status").read()
            cap = int(next(l for l in status.splitlines() if l.startswith("CapEff")).split()[1], 16)
            findings["cap_sys_admin"] = bool(cap >> 21 & 1)
            findings["cap_sys_ptrace"] = bool(cap >> 19 & 1)
        except (OSError, StopIteration, ValueError):
            pass
        findings["docker_socket"] = os.access("/var/run/docker.sock", os.W_OK)
        try:
            findings["host_pid_namespace"] = os.path.exists("/proc/1/cmdline") and b"systemd" in open("/proc/1/cmdline", "rb").read()
        except OSError:
            findings["host_pid_namespace"] = False
        return findings


class AdvancedMonitor:
    """Resource watcher: samples CPU, memory and open files of this process and reports threshold crossings."""

    def __init__(self, max_rss_mb: float = 0.0, max_open_files: int = 0):
        self.max_rss_mb, self.max_open_files = max_rss_mb, max_open_files

    def sample(self) -> dict:
        import psutil
        p = psutil.Process()
        s = {"rss_mb": p.memory_info().rss / 2 ** 20, "cpu_percent": p.cpu_percent(interval=None), "open_files": len(p.open_files()),
             "threads": p.num_threads()}
        s["alerts"] = [k for k, lim in (("rss_mb", self.max_rss_mb), ("open_files", self.max_open_files)) if lim and s[k] > lim]
        return s


class TransportSecurity:
    """TLS server context with modern defaults (TLS 1.2+, no compression) for the HTTP front-ends."""

    def __init__(self, certfile: str, keyfile: str, client_ca: Optional[str] = None):
        self.certfile, self.keyfile, self.client_ca = certfile, keyfile, client_ca

    def context(self):
        import ssl
        ctx = ssl.SSLContext(ssl.PROTOCOL_TLS_SERVER)
        ctx.minimum_version = ssl.TLSVersion.TLSv1_2
        ctx.options |= ssl.OP_NO_COMPRESSION
        ctx.load_cert_chain(self.certfile, self.keyfile)
        if self.client_ca:   # mutual TLS
            ctx.verify_mode = ssl.CERT_REQUIRED
            ctx.load_verify_locations(self.client_ca)
        return ctx


class RemoteAPIAuditBackend(_svc.AuditLogger):
    """Audit chain that also posts each record to a collector URL; delivery failures are counted, never raised."""

    def __init__(self, path: str, url: str, timeout: float = 2.0):
        super().__init__(path)
        self.url, self.timeout, self.failed = url, timeout, 0

    def log(self, actor, action, **details):
        import urllib.request
        h = super().log(actor, action, **details)
        try:
            req = urllib.request.Request(self.url, data=json.dumps({"actor": actor, "action": action, "hash": h}).encode(),
                                         headers={"Content-Type": "application/json"}, method="POST")
            urllib.request.urlopen(req, timeout=self.timeout).read()
        except Exception:
            self.failed += 1
        return h




ObfuscationPipeline = _lazy("security.obfuscation", "ObfuscationPipeline")
ObfuscationConfig = _lazy("security.obfuscation", "ObfuscationConfig")


class _ProgramPass:
    """One obfuscation pass over an NPE program; ``apply(program, **options)`` returns the transformed program."""

    fn_name = ""

    def __init__(self, **options):
        self.options = options

    def apply(self, program, **options):
        from .security import obfuscation
        return getattr(obfuscation, self.fn_name)(program, **dict(self.options, **options))

    __call__ = apply


class InstructionSubstitution(_ProgramPass):
    fn_name = "substitute_instructions"


class OpaquePredicate(_ProgramPass):
    fn_name = "insert_opaque_predicates"


class StringEncryption(_ProgramPass):
    """Seals a program (encrypts and authenticates its serialised form)."""

    fn_name = "seal_program"


# ---------------------------------------------------------------------------------------------- late additions
from .utils.net import RDMA  # noqa: E402,F401

ABOOTPartition = _svc.ABSlots

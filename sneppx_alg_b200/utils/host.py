"""ctypes bindings of the small C++ host components: BPE tokenizer, model factory, serving batch core, edge runtime,
CPU oracles, memory pool."""
from __future__ import annotations

import ctypes as C
import json
import struct
from typing import List

import numpy as np

from .. import _build


def _L():
    L = _build.load_host()
    if not getattr(L, "_misc_ready", False):
        for f in ("sx_tok_create", "sx_sc_create", "sx_edge_arena_create", "sx_edge_load", "sx_pool_create",
                  "sx_threadpool_create", "sx_edge_arena_alloc", "sx_pool_alloc"):
            getattr(L, f).restype = C.c_void_p
        L.sx_tok_train.argtypes = [C.c_void_p, C.c_char_p, C.c_longlong, C.c_int]
        L.sx_tok_encode.argtypes = [C.c_void_p, C.c_char_p, C.c_longlong, C.c_void_p, C.c_longlong]
        L.sx_tok_encode.restype = C.c_longlong
        L.sx_tok_decode.argtypes = [C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p, C.c_longlong]
        L.sx_tok_decode.restype = C.c_longlong
        for f in ("sx_tok_destroy", "sx_tok_vocab_size", "sx_sc_destroy", "sx_sc_pending", "sx_sc_breaker_allow",
                  "sx_sc_breaker_state", "sx_edge_free", "sx_pool_destroy"):
            getattr(L, f).argtypes = [C.c_void_p]
        L.sx_tok_save.argtypes = L.sx_tok_load.argtypes = [C.c_void_p, C.c_char_p]
        L.sx_sc_create.argtypes = [C.c_int, C.c_double]
        L.sx_sc_submit.argtypes = [C.c_void_p, C.c_longlong, C.c_int]
        L.sx_sc_next_batch.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        L.sx_sc_record.argtypes = [C.c_void_p, C.c_double, C.c_int]
        L.sx_sc_metrics.argtypes = [C.c_void_p, C.c_void_p]
        L.sx_sc_route.argtypes = [C.c_char_p, C.c_void_p, C.c_int]
        L.sx_sc_breaker_config.argtypes = [C.c_void_p, C.c_int, C.c_double]
        L.sx_factory_config_from_name.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
        L.sx_factory_extend_context.argtypes = [C.c_char_p, C.c_int, C.c_char_p, C.c_char_p, C.c_int]
        L.sx_factory_search.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
        L.sx_edge_load.argtypes = [C.c_char_p]
        L.sx_edge_run.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        L.sx_edge_max_width.argtypes = [C.c_void_p, C.c_int]
        L.sx_oracle_ssd.argtypes = [C.c_void_p] * 7 + [C.c_int] * 6
        L.sx_oracle_router.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        L.sx_oracle_adamw.argtypes = [C.c_void_p] * 4 + [C.c_longlong] + [C.c_float] * 5 + [C.c_int]
        L._misc_ready = True
    return L


class BPETokenizer:
    def __init__(self):
        self._h = _L().sx_tok_create()

    def train(self, text: str, vocab_size: int) -> int:
        b = text.encode("utf-8")
        return _L().sx_tok_train(self._h, b, len(b), vocab_size)

    @property
    def vocab_size(self):
        return _L().sx_tok_vocab_size(self._h)

    def encode(self, text: str) -> List[int]:
        b = text.encode("utf-8")
        out = (C.c_int * max(1, len(b)))()
        n = _L().sx_tok_encode(self._h, b, len(b), out, len(b))
        return list(out[:n])

    def decode(self, ids: List[int]) -> str:
        arr = (C.c_int * max(1, len(ids)))(*ids)
        cap = 64 + 16 * len(ids)
        while True:
            buf = C.create_string_buffer(cap)
            n = _L().sx_tok_decode(self._h, arr, len(ids), buf, cap)
            if n >= 0:
                return buf.raw[:n].decode("utf-8", errors="replace")
            cap = -n + 1

    def save(self, path):
        return _L().sx_tok_save(self._h, path.encode())

    def load(self, path):
        rc = _L().sx_tok_load(self._h, path.encode())
        if rc:
            raise IOError(f"cannot load tokenizer {path} ({rc})")
        return self


def factory_config(name: str, extend_to: int = 0, method: str = "ntk") -> dict:
    buf = C.create_string_buffer(4096)
    n = (_L().sx_factory_extend_context(name.encode(), extend_to, method.encode(), buf, 4096) if extend_to
         else _L().sx_factory_config_from_name(name.encode(), buf, 4096))
    if n < 0:
        raise KeyError(name)
    return json.loads(buf.value.decode())


def factory_search(q: str) -> List[str]:
    buf = C.create_string_buffer(8192)
    _L().sx_factory_search(q.encode(), buf, 8192)
    return [s for s in buf.value.decode().split("\n") if s]


class ServingCore:
    def __init__(self, max_batch=32, timeout_ms=2.0):
        self._h = _L().sx_sc_create(max_batch, timeout_ms)

    def submit(self, rid: int, priority: int = 0):
        _L().sx_sc_submit(self._h, rid, priority)

    def next_batch(self, force=False, cap=256) -> List[int]:
        out = (C.c_longlong * cap)()
        n = _L().sx_sc_next_batch(self._h, out, cap, int(force))
        return list(out[:n])

    def record(self, latency_s: float, ok=True):
        _L().sx_sc_record(self._h, latency_s, int(ok))

    def metrics(self):
        out = (C.c_double * 6)()
        _L().sx_sc_metrics(self._h, out)
        return dict(zip(("p50", "p95", "p99", "rps", "requests", "errors"), out))

    @staticmethod
    def route(request_id: str, weights: List[float]) -> int:
        w = (C.c_double * len(weights))(*weights)
        return _L().sx_sc_route(request_id.encode(), w, len(weights))

    def breaker_config(self, fail_threshold=5, cooldown_ms=1000.0):
        _L().sx_sc_breaker_config(self._h, fail_threshold, cooldown_ms)

    def breaker_allow(self) -> bool:
        return bool(_L().sx_sc_breaker_allow(self._h))


def write_edge_model(path: str, layers):
    """layers: list of ('matmul', W [in, out]) | ('bias', b [out]) | ('relu',)."""
    with open(path, "wb") as f:
        f.write(b"EDGE" + struct.pack("<II", 1, len(layers)))
        for l in layers:
            if l[0] == "matmul":
                w = np.ascontiguousarray(l[1], dtype=np.float32)
                f.write(struct.pack("<III", 1, w.shape[0], w.shape[1]) + w.tobytes())
            elif l[0] == "bias":
                b = np.ascontiguousarray(l[1], dtype=np.float32)
                f.write(struct.pack("<III", 3, 1, b.shape[0]) + b.tobytes())
            else:
                f.write(struct.pack("<III", 2, 0, 0))


class EdgeModel:
    def __init__(self, path: str):
        self._h = _L().sx_edge_load(path.encode())
        if not self._h:
            raise IOError(f"cannot load edge model {path}")

    def run(self, x: np.ndarray, max_width: int = 4096) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        max_width = max(max_width, _L().sx_edge_max_width(self._h, x.shape[1]))  # never smaller than the model needs
        y = np.zeros((x.shape[0], max_width), dtype=np.float32)
        d = _L().sx_edge_run(self._h, x.ctypes.data, x.shape[0], x.shape[1], y.ctypes.data, None)
        if d < 0:
            raise ValueError("shape mismatch in edge model")
        return y.reshape(-1)[: x.shape[0] * d].reshape(x.shape[0], d)


def oracle_ssd(x, dt, A, Bm, Cm, D):
    x, dt, A, Bm, Cm, D = [np.ascontiguousarray(t, dtype=np.float32) for t in (x, dt, A, Bm, Cm, D)]
    B, L, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    y = np.zeros_like(x)
    _L().sx_oracle_ssd(x.ctypes.data, dt.ctypes.data, A.ctypes.data, Bm.ctypes.data, Cm.ctypes.data, D.ctypes.data,
                       y.ctypes.data, B, L, H, P, G, N)
    return y


def oracle_router(logits, k):
    lg = np.ascontiguousarray(logits, dtype=np.float32)
    T, E = lg.shape
    idx = np.zeros((T, k), dtype=np.int32)
    w = np.zeros((T, k), dtype=np.float32)
    _L().sx_oracle_router(lg.ctypes.data, T, E, k, idx.ctypes.data, w.ctypes.data)
    return idx, w


def oracle_adamw(p, m, v, g, lr, b1, b2, eps, wd, step):
    _L().sx_oracle_adamw(p.ctypes.data, m.ctypes.data, v.ctypes.data, g.ctypes.data, p.size, lr, b1, b2, eps, wd, step)
    return p

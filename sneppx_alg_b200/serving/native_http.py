"""C++ HTTP front-end (``csrc/host/http_server.cpp``) with Python route handlers.

The socket work (accept, parse, route match, Bearer check, counters) runs in C++ worker threads; a handler is only
entered, under the GIL, for routes that need the engine. ``serve_engine`` publishes the reference's C REST surface
(``net/http/http_api.c:326-329``: ``/v1/health``, ``/v1/models``, ``/v1/models/{id}``, ``/v1/generate``) on top of any
object with ``generate(prompt, **sampling) -> dict``; the FastAPI application in ``serving/server.py`` remains the full
API (streaming, chat, admin).
"""
from __future__ import annotations

import ctypes as C
import json
import threading
from typing import Callable, Dict, Optional

from .. import _build

_CB = C.CFUNCTYPE(C.c_longlong, C.c_char_p, C.c_char_p, C.c_char_p, C.POINTER(C.c_char), C.c_longlong,
                  C.POINTER(C.c_char), C.c_longlong, C.POINTER(C.c_int))


def _L():
    L = _build.load_host()
    if not getattr(L, "_http_ready", False):
        L.sx_http_create.restype = C.c_void_p
        L.sx_http_create.argtypes = [C.c_char_p, C.c_longlong]
        L.sx_http_add_route.argtypes = [C.c_void_p, C.c_char_p, C.c_char_p, C.c_int, C.c_char_p, _CB]
        L.sx_http_start.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.sx_http_start_on.argtypes = [C.c_void_p, C.c_char_p, C.c_int, C.c_int]
        L.sx_http_stop.argtypes = [C.c_void_p]
        L.sx_http_route_hits.argtypes = [C.c_void_p, C.c_int]
        L.sx_http_route_hits.restype = C.c_longlong
        L._http_ready = True
    return L


class HTTPError(Exception):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status, self.message = status, message


class NativeHttpServer:
    """``route`` handlers take ``(params: dict, body: bytes)`` and return a JSON-serialisable object, ``bytes``, or a
    ``(status, object)`` pair; raising ``HTTPError`` sets the status. Register every route before ``start``."""

    def __init__(self, token: str = "", max_body: int = 8 << 20):
        self._h = _L().sx_http_create(token.encode(), max_body)
        self._keep = []  # callback objects must outlive the server
        self.port: Optional[int] = None
        self._routes: Dict[str, int] = {}
        self._held: Dict[int, tuple] = {}  # worker thread id -> (status, body) awaiting a larger buffer

    def static(self, method: str, pattern: str, payload, public: bool = False):
        body = payload if isinstance(payload, (bytes, str)) else json.dumps(payload)
        body = body.encode() if isinstance(body, str) else body
        self._routes[f"{method} {pattern}"] = _L().sx_http_add_route(self._h, method.encode(), pattern.encode(), int(public),
                                                                    body, _CB())

    def route(self, method: str, pattern: str, public: bool = False):
        def deco(fn: Callable):
            def cb(_m, _p, params, body, blen, out, cap, status):
                held = self._held.pop(threading.get_ident(), None)
                if held is not None:  # second call for a response that did not fit: hand over what the first call made
                    status[0], data = held
                    if len(data) > cap:
                        return -len(data)
                    C.memmove(out, data, len(data))
                    return len(data)
                try:
                    res = fn(json.loads(params.decode()), C.string_at(body, blen) if blen else b"")
                    if isinstance(res, tuple):
                        status[0], res = int(res[0]), res[1]
                    data = res if isinstance(res, bytes) else json.dumps(res).encode()
                except HTTPError as e:
                    status[0], data = e.status, json.dumps({"error": e.message}).encode()
                except Exception as e:  # a handler bug must not take the server thread down
                    status[0], data = 500, json.dumps({"error": f"{type(e).__name__}: {e}"}).encode()
                if len(data) > cap:
                    self._held[threading.get_ident()] = (status[0], data)  # the handler must not run twice
                    return -len(data)
                C.memmove(out, data, len(data))
                return len(data)

            c = _CB(cb)
            self._keep.append(c)
            self._routes[f"{method} {pattern}"] = _L().sx_http_add_route(self._h, method.encode(), pattern.encode(),
                                                                        int(public), None, c)
            return fn
        return deco

    def start(self, port: int = 0, workers: int = 4, host: str = "127.0.0.1") -> int:
        """Binds `host` (dotted IPv4; "0.0.0.0" for every interface) and starts the accept and worker threads."""
        p = _L().sx_http_start_on(self._h, host.encode(), port, workers)
        if p < 0:
            raise OSError(f"cannot bind {host}:{port}")
        self.port = p
        return p

    def hits(self, method: str, pattern: str) -> int:
        return _L().sx_http_route_hits(self._h, self._routes[f"{method} {pattern}"])

    def stop(self):
        if self._h:
            _L().sx_http_stop(self._h)
            self._h = None


def serve_engine(engine, models: Dict[str, dict], token: str = "", port: int = 0, workers: int = 4,
                 host: str = "127.0.0.1") -> NativeHttpServer:
    """Starts the REST surface of the reference's C API in front of `engine`. ``models``: id -> description."""
    srv = NativeHttpServer(token)
    srv.static("GET", "/v1/health", {"status": "ok"}, public=True)
    srv.static("GET", "/v1/models", {"models": [dict(id=k, **v) for k, v in models.items()]})

    @srv.route("GET", "/v1/models/{id}")
    def _model(params, _body):
        if params["id"] not in models:
            raise HTTPError(404, f"unknown model {params['id']}")
        return dict(id=params["id"], **models[params["id"]])

    @srv.route("POST", "/v1/generate")
    def _generate(_params, body):
        try:
            req = json.loads(body or b"{}")
        except (ValueError, RecursionError):      # RecursionError: thousands of nested brackets
            raise HTTPError(400, "body is not JSON")
        if not isinstance(req, dict) or not isinstance(req.get("prompt"), str):
            raise HTTPError(400, "prompt (string) is required")
        try:
            n = int(req.get("max_new_tokens", 32))
        except (TypeError, ValueError, OverflowError):
            raise HTTPError(400, "max_new_tokens must be an integer")
        if not 0 < n <= 4096:
            raise HTTPError(400, "max_new_tokens must be in 1..4096")
        if req.get("model") and req["model"] not in models:
            raise HTTPError(404, f"unknown model {req['model']}")
        kw = {k: req[k] for k in ("do_sample", "temperature", "top_k", "top_p", "repetition_penalty", "stop_strings") if k in req}
        return engine.generate(req["prompt"], max_new_tokens=n, **kw)

    srv.start(port, workers, host)
    return srv


class TextEngine:
    """Adapter from text requests to the continuous-batching engine: tokenise, submit to the engine's worker thread,
    wait, filter, and return the ``GenerateResponse`` fields of the reference schema (inference_server.py:67-150)."""

    def __init__(self, model, tokenizer=None, model_id: str = "default", **engine_kwargs):
        from ..security.ai_filter import OutputVerifier, PromptFilter
        from .llm_engine import LLMEngine
        from .server import ByteTokenizer, EngineWorker
        self.model_id = model_id
        self.tok = tokenizer or ByteTokenizer(model.config.vocab_size)
        self.worker = EngineWorker(LLMEngine(model, **engine_kwargs))
        self.filter, self.verifier = PromptFilter(), OutputVerifier()

    def generate(self, prompt: str, max_new_tokens: int = 32, **sampling) -> dict:
        import time

        from .llm_engine import SamplingParams
        chk = self.filter.check(prompt)
        if not chk.allowed:
            raise HTTPError(400, "prompt rejected: " + "; ".join(chk.reasons))
        from .generation import make_stop_fn, truncate_at_stop
        stops = sampling.pop("stop_strings", None)
        ids = self.tok.encode(chk.sanitized)
        sp = SamplingParams(max_new_tokens=max_new_tokens, stop_fn=make_stop_fn(self.tok, stops), **sampling)
        rid, ev = self.worker.submit(ids, sp)
        if not ev.wait(timeout=600):
            raise HTTPError(503, "generation timed out")
        req = self.worker.result(rid)
        text = self.verifier.verify(truncate_at_stop(self.tok.decode(req.output), stops)).sanitized
        return {"generated_text": text, "token_ids": req.output, "prompt_tokens": len(ids), "completion_tokens": len(req.output),
                "total_tokens": len(ids) + len(req.output), "model": self.model_id, "created": int(time.time())}

    def stop(self):
        self.worker.stop()

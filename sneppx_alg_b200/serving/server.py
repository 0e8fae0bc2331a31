"""REST front-end: ``/v1/generate`` family, OpenAI-shaped chat completions, health / readiness, metrics, model
management, admin API keys. Endpoint set and JSON schemas follow the reference server
(interface_bindings/inference_server.py:67-150 schemas, :372-905 routes; C routes net/http/http_api.c:326-329).
Generation runs through the paged continuous-batching engine: concurrent HTTP requests are merged into one
decode batch by a background scheduler thread."""


import asyncio
import json
import secrets
import threading
import time
import uuid
from typing import Dict, List, Optional

from ..security.ai_filter import OutputVerifier, PromptFilter
from .llm_engine import LLMEngine, SamplingParams
from .serving_engine import MetricsCollector, ServingEngine


class ByteTokenizer:
    """Fallback tokenizer of the reference server: code point modulo vocabulary (inference_server.py:475-478)."""

    def __init__(self, vocab_size: int):
        self.vocab_size = vocab_size

    def encode(self, text: str) -> List[int]:
        return [ord(c) % self.vocab_size for c in text] or [0]

    def decode(self, ids: List[int]) -> str:
        # code points that cannot be encoded as UTF-8 on their own (surrogates) print as "?" like control characters
        return "".join(chr(i) if (32 <= i < 0xD800 or 0xE000 <= i < 0x110000) else "?" for i in ids)


class EngineWorker:
    """Owns one LLMEngine and steps it on a background thread; HTTP handlers submit and await futures. Submissions
    only append to a list under a lock that is never held across an engine step (a handler running on the event loop
    must not wait for a step, and an unfair lock would let the stepping thread starve it); the stepping thread moves
    them into the engine at the start of its next iteration, so request ids are handed out here."""

    def __init__(self, engine: LLMEngine):
        self.engine = engine
        self._lock = threading.Lock()
        self._events: Dict[int, threading.Event] = {}
        self._callbacks: Dict[int, object] = {}
        self._pending: list = []
        self._next_rid = 0
        self._stop = False
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def _fire_finished(self):
        with self._lock:
            done = [rid for rid in self._events if rid in self.engine.finished or rid in self.engine.failed]
            fired = [(self._events.pop(rid), self._callbacks.pop(rid, None)) for rid in done]
        for ev, cb in fired:
            ev.set()
            if cb is not None:
                cb()

    def _loop(self):
        try:
            dev = next(self.engine.runner.model.parameters()).device
            if dev.type == "cuda":
                import torch
                torch.cuda.set_device(dev)       # a new thread starts on device 0
        except (AttributeError, StopIteration):
            pass
        while not self._stop:
            with self._lock:
                new, self._pending = self._pending, []
            for prompt, sp, on_token, rid in new:
                got = self.engine.submit(prompt, sp, on_token=on_token)
                if got != rid:
                    raise RuntimeError("request ids diverged: something else submitted to this engine")
            if self.engine.has_work():
                self.engine.step()
                self._fire_finished()
            else:
                time.sleep(0.001)

    def submit(self, prompt_ids, params, on_token=None, on_done=None):
        """``on_done``: called (on the engine thread) when the request has finished; lets an event loop await the
        result without parking a thread per request."""
        ev = threading.Event()
        with self._lock:
            rid = self._next_rid
            self._next_rid += 1
            self._pending.append((list(prompt_ids), params, on_token, rid))
            self._events[rid] = ev
            if on_done is not None:
                self._callbacks[rid] = on_done
        return rid, ev

    def result(self, rid):
        return self.engine.finished.pop(rid)

    def stop(self):
        self._stop = True


class TPEngineWorker(EngineWorker):
    """Tensor-parallel form of the worker. Every rank of ``group`` owns an ``LLMEngine`` over its shard of the model;
    the engines only stay consistent if all of them see the same requests in the same order and step together. The
    leader (group rank 0) takes submissions from the HTTP handlers; once per loop iteration it broadcasts the new
    ones (a three-word header, then the prompts and sampling parameters as JSON when there are any) and every rank
    submits them and takes one engine step. The other ranks run ``follow()``, which returns when the leader stops.
    Requests with a ``stop_fn`` are refused: the callable lives on the leader only."""

    def __init__(self, engine: LLMEngine, group):
        import torch.distributed as dist
        self.group = group
        self.leader = dist.get_rank(group) == 0
        self.src = dist.get_global_rank(group, 0)
        self.dev = next(engine.runner.model.parameters()).device
        self._pending: list = []
        self._next_rid = 0
        if self.leader:
            super().__init__(engine)     # starts the loop thread
        else:
            self.engine, self._stop = engine, False
            self._lock, self._events, self._callbacks = threading.Lock(), {}, {}

    def _exchange(self, items, stop):
        import torch
        import torch.distributed as dist
        payload = json.dumps(items).encode() if (self.leader and items) else b""
        hdr = torch.tensor([len(items), len(payload), int(stop)] if self.leader else [0, 0, 0], dtype=torch.int64,
                           device=self.dev)
        dist.broadcast(hdr, self.src, group=self.group)
        n, nbytes, stop = hdr.tolist()
        if nbytes:
            if self.leader:
                buf = torch.frombuffer(bytearray(payload), dtype=torch.uint8).to(self.dev)
            else:
                buf = torch.empty(nbytes, dtype=torch.uint8, device=self.dev)
            dist.broadcast(buf, self.src, group=self.group)
            if not self.leader:
                items = json.loads(buf.cpu().numpy().tobytes().decode())
        return items if n else [], bool(stop)

    def _loop(self):
        from dataclasses import asdict
        if self.dev.type == "cuda":
            import torch
            torch.cuda.set_device(self.dev)      # the leader's loop runs on a thread of its own
        while True:
            with self._lock:
                new, self._pending = self._pending, []
                stop = self._stop
            items, stop = self._exchange([(p, asdict(sp)) for p, sp, _, _ in new] if self.leader else [], stop)
            for i, (prompt, pd) in enumerate(items):
                pd["stop_token_ids"] = tuple(pd.get("stop_token_ids", ()))
                rid = self.engine.submit(prompt, SamplingParams(**pd), on_token=new[i][2] if self.leader else None)
                if self.leader and rid != new[i][3]:
                    raise RuntimeError("request ids of the tensor-parallel engines diverged")
            if stop:
                return
            if self.engine.has_work():
                self.engine.step()
                self._fire_finished()
            elif self.leader:
                time.sleep(0.002)

    follow = _loop

    def submit(self, prompt_ids, params, on_token=None, on_done=None):
        if params.stop_fn is not None:
            raise ValueError("stop strings / stop_fn are not supported by tensor-parallel serving")
        return super().submit(prompt_ids, params, on_token=on_token, on_done=on_done)

    def stop(self):
        self._stop = True
        if self.leader:
            self.thread.join(30)


def tp_follow(model, engine_kwargs: dict):
    """What the ranks other than group rank 0 run while rank 0 serves HTTP: build the same engine and mirror it."""
    eng = LLMEngine(model, **engine_kwargs)
    TPEngineWorker(eng, engine_kwargs["tp_group"]).follow()


def create_app(models: Dict[str, dict], default_model: Optional[str] = None, api_keys: Optional[set] = None,
               admin_key: Optional[str] = None):
    """models: {model_id: {"model": LlamaForCausalLM, "tokenizer": obj with encode/decode (optional), "engine_kwargs": {...}}}"""
    from fastapi import FastAPI, Header, HTTPException
    from fastapi.responses import PlainTextResponse, StreamingResponse
    from pydantic import BaseModel, Field

    app = FastAPI(title="sneppx serving", version="0.1.0")
    metrics = MetricsCollector()
    control = ServingEngine()
    prompt_filter, verifier = PromptFilter(), OutputVerifier()
    workers: Dict[str, EngineWorker] = {}
    toks = {}
    keys = set(api_keys or [])
    default_model = default_model or next(iter(models))
    for mid, spec in models.items():
        eng = LLMEngine(spec["model"], **spec.get("engine_kwargs", {}))
        tpg = spec.get("engine_kwargs", {}).get("tp_group")
        workers[mid] = TPEngineWorker(eng, tpg) if tpg is not None else EngineWorker(eng)
        toks[mid] = spec.get("tokenizer") or ByteTokenizer(spec["model"].config.vocab_size)
        control.register_model(mid, "v1", handler=lambda *a, **k: None)
        control.deploy(mid, "v1", 1.0)
    app.state.workers, app.state.metrics, app.state.control = workers, metrics, control

    class GenerateRequest(BaseModel):
        prompt: str = ""
        prompt_token_ids: Optional[List[int]] = None      # already tokenised prompt (takes precedence over `prompt`)
        max_new_tokens: int = Field(64, ge=1, le=4096)
        do_sample: bool = False
        temperature: float = 1.0
        top_k: int = 0
        top_p: float = 1.0
        repetition_penalty: float = 1.0
        num_beams: int = 1
        stop_strings: Optional[List[str]] = None
        model: Optional[str] = None

    class BatchRequest(BaseModel):
        prompts: List[str]
        max_new_tokens: int = Field(64, ge=1, le=4096)
        do_sample: bool = False
        temperature: float = 1.0
        top_k: int = 0
        top_p: float = 1.0
        model: Optional[str] = None

    class ChatMessage(BaseModel):
        role: str
        content: str

    class ChatRequest(BaseModel):
        messages: List[ChatMessage]
        model: Optional[str] = None
        max_tokens: int = 64
        temperature: float = 1.0
        top_p: float = 1.0
        stream: bool = False

    def auth(authorization: Optional[str]):
        if not keys:
            return
        tok = (authorization or "").removeprefix("Bearer ").strip()
        if tok not in keys and tok != admin_key:
            raise HTTPException(401, "invalid API key")

    def params_of(r) -> SamplingParams:
        return SamplingParams(max_new_tokens=r.max_new_tokens, do_sample=r.do_sample, temperature=r.temperature,
                              top_k=r.top_k, top_p=r.top_p, repetition_penalty=getattr(r, "repetition_penalty", 1.0))

    async def run_one(mid: str, prompt: str, sp: SamplingParams, stop_strings=None, token_ids=None):
        if mid not in workers:
            raise HTTPException(404, f"unknown model '{mid}'")
        if stop_strings:
            from .generation import make_stop_fn
            sp.stop_fn = make_stop_fn(toks[mid], stop_strings)
        t0 = time.perf_counter()
        if token_ids is not None:
            vocab = models[mid]["model"].config.vocab_size
            if not token_ids or any((not isinstance(t, int)) or t < 0 or t >= vocab for t in token_ids):
                raise HTTPException(400, {"error": "prompt_token_ids must be non-empty ids inside the vocabulary"})
            ids = list(token_ids)
        else:
            chk = prompt_filter.check(prompt)
            if not chk.allowed:
                raise HTTPException(400, {"error": "prompt rejected", "reasons": chk.reasons})
            ids = toks[mid].encode(chk.sanitized)
        loop = asyncio.get_running_loop()
        done = loop.create_future()
        rid, ev = workers[mid].submit(ids, sp, on_done=lambda: loop.call_soon_threadsafe(
            lambda: done.done() or done.set_result(None)))
        await done
        why = workers[mid].engine.failed.pop(rid, None)
        req = workers[mid].result(rid)
        if why is not None:
            raise HTTPException(413, {"error": why})
        text = toks[mid].decode(req.output)
        if stop_strings:
            from .generation import truncate_at_stop
            text = truncate_at_stop(text, stop_strings)
        text = verifier.verify(text).sanitized
        metrics.record(time.perf_counter() - t0, True, len(ids), len(req.output),
                       (req.first_token_time - req.arrival) if req.first_token_time else None)
        return {"generated_text": text, "token_ids": req.output, "prompt_tokens": len(ids),
                "completion_tokens": len(req.output), "total_tokens": len(ids) + len(req.output), "model": mid,
                "created": int(time.time()),
                "ttft_s": (req.first_token_time - req.arrival) if req.first_token_time else None}

    @app.get("/v1/health")
    def health():
        return {"status": "ok", "models": list(workers), "uptime_s": metrics.snapshot()["uptime_s"]}

    @app.get("/healthz")
    def healthz():
        return {"status": "ok"}

    @app.get("/readyz")
    def readyz():
        return {"ready": bool(workers)}

    @app.get("/metrics")
    def metrics_ep(format: str = "prometheus"):
        if format == "json":
            return metrics.snapshot()
        return PlainTextResponse(metrics.prometheus())

    @app.get("/v1/models")
    def list_models():
        return {"data": [{"id": m, "object": "model", "versions": control.list_models().get(m, {})} for m in workers]}

    @app.get("/v1/models/{model_id}")
    def get_model(model_id: str):
        if model_id not in workers:
            raise HTTPException(404, "unknown model")
        cfg = models[model_id]["model"].config
        return {"id": model_id, "config": cfg.to_dict(), "versions": control.list_models().get(model_id, {})}

    @app.get("/v1/models/{model_id}/card")
    def get_model_card(model_id: str):
        """Model card of a served model: the one passed in its spec (``card``), else one derived from the module."""
        if model_id not in workers:
            raise HTTPException(404, "unknown model")
        from dataclasses import asdict
        from ..hub.model_card import ModelCard
        card = models[model_id].get("card") or ModelCard.from_model(models[model_id]["model"], model_id, model_type="causal-lm")
        return asdict(card)

    @app.get("/v1/models/{model_id}/versions")
    def get_versions(model_id: str):
        return control.list_models().get(model_id, {})

    @app.post("/v1/deploy")
    def deploy(body: dict, authorization: Optional[str] = Header(None)):
        auth(authorization)
        control.deploy(body["model"], body.get("version", "v1"), float(body.get("weight", 1.0)))
        return {"ok": True}

    @app.post("/v1/traffic")
    def traffic(body: dict, authorization: Optional[str] = Header(None)):
        auth(authorization)
        control.set_traffic(body["model"], body["weights"])
        return {"ok": True}

    @app.post("/v1/generate")
    async def generate_ep(r: GenerateRequest, authorization: Optional[str] = Header(None)):
        auth(authorization)
        return await run_one(r.model or default_model, r.prompt, params_of(r), r.stop_strings, r.prompt_token_ids)

    @app.post("/v1/generate/batch")
    async def generate_batch(r: BatchRequest, authorization: Optional[str] = Header(None)):
        auth(authorization)
        mid = r.model or default_model
        sp = SamplingParams(max_new_tokens=r.max_new_tokens, do_sample=r.do_sample, temperature=r.temperature,
                            top_k=r.top_k, top_p=r.top_p)
        return {"results": list(await asyncio.gather(*[run_one(mid, p, sp) for p in r.prompts]))}

    @app.post("/v1/generate/continuous-batch")
    async def generate_cb(r: BatchRequest, authorization: Optional[str] = Header(None)):
        return await generate_batch(r, authorization)

    @app.post("/v1/generate/stream")
    async def generate_stream(r: GenerateRequest, authorization: Optional[str] = Header(None)):
        auth(authorization)
        mid = r.model or default_model
        chk = prompt_filter.check(r.prompt)
        if not chk.allowed:
            raise HTTPException(400, {"error": "prompt rejected", "reasons": chk.reasons})
        q: asyncio.Queue = asyncio.Queue()
        loop = asyncio.get_running_loop()
        ids = toks[mid].encode(chk.sanitized)
        rid, ev = workers[mid].submit(ids, params_of(r), on_token=lambda _rid, t: loop.call_soon_threadsafe(q.put_nowait, t))

        async def events():
            n = 0
            while n < r.max_new_tokens:
                try:
                    t = await asyncio.wait_for(q.get(), timeout=0.05)
                except asyncio.TimeoutError:
                    if ev.is_set() and q.empty():
                        break
                    continue
                n += 1
                yield f"data: {json.dumps({'token_id': t, 'text': toks[mid].decode([t])})}\n\n"
            yield "data: [DONE]\n\n"

        return StreamingResponse(events(), media_type="text/event-stream")

    @app.post("/v1/chat/completions")
    async def chat(r: ChatRequest, authorization: Optional[str] = Header(None)):
        auth(authorization)
        prompt = "\n".join(f"{m.role}: {m.content}" for m in r.messages) + "\nassistant:"
        sp = SamplingParams(max_new_tokens=r.max_tokens, do_sample=r.temperature > 0 and r.temperature != 1.0,
                            temperature=r.temperature, top_p=r.top_p)
        out = await run_one(r.model or default_model, prompt, sp)
        return {"id": "chatcmpl-" + uuid.uuid4().hex[:12], "object": "chat.completion", "created": out["created"],
                "model": out["model"],
                "choices": [{"index": 0, "message": {"role": "assistant", "content": out["generated_text"]},
                             "finish_reason": "length"}],
                "usage": {"prompt_tokens": out["prompt_tokens"], "completion_tokens": out["completion_tokens"],
                          "total_tokens": out["total_tokens"]}}

    @app.post("/v1/models/quantize")
    def quantize(body: dict, authorization: Optional[str] = Header(None)):
        auth(authorization)
        from ..ops.quant import quantize_model_
        mid = body.get("model", default_model)
        quantize_model_(models[mid]["model"], body.get("mode", "fp8"))
        return {"ok": True, "model": mid, "mode": body.get("mode", "fp8")}

    @app.post("/v1/admin/keys")
    def create_key(authorization: Optional[str] = Header(None)):
        if admin_key and (authorization or "").removeprefix("Bearer ").strip() != admin_key:
            raise HTTPException(403, "admin key required")
        k = "sk-" + secrets.token_hex(16)
        keys.add(k)
        return {"api_key": k}

    @app.delete("/v1/admin/keys/{key}")
    def delete_key(key: str, authorization: Optional[str] = Header(None)):
        if admin_key and (authorization or "").removeprefix("Bearer ").strip() != admin_key:
            raise HTTPException(403, "admin key required")
        keys.discard(key)
        return {"ok": True}

    return app

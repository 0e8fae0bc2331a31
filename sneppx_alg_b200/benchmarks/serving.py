"""Serving benchmark: N concurrent requests through the continuous-batching engine (the engine behind ``/v1/generate``),
reporting output tokens per second and time to first token.

``python -m sneppx_alg_b200.benchmarks.serving [--model llama3-8b] [--requests 64] [--prompt-len 2048] [--new-tokens 256]
[--quantize none|fp8|int4] [--http] [--out file.json]``
``--http`` drives the same workload through the HTTP front-end: the FastAPI application is served by uvicorn on
127.0.0.1 and every request is a ``POST /v1/generate`` carrying its prompt as token ids, all sent at once from client
threads; TTFT is the server's figure for each request (submission to first token), throughput is client wall clock.
Under ``torch.distributed.run`` with N ranks the engine runs tensor-parallel over all of them (``TPLlamaPagedRunner``).

The default workload is the serving configuration of the baseline list: 64 concurrent requests, prompts of 2048
random token ids, 256 greedy decode tokens each, random-init weights (the reference's ``benchmarks/serving_benchmark.py``
compares static and continuous batching on a dummy model that returns random logits; here the model is real). All
requests are submitted at time zero; TTFT of a request is measured from submission to its first sampled token, so it
includes the queueing behind earlier prefills. One GPU; the prompts are distinct, so the prefix cache gives no help.
Timing is wall clock around ``run_until_done`` with a device synchronisation on both sides (the loop reads one token
id per request back every step, which is part of serving).
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import torch


def run(model, requests=64, prompt_len=2048, new_tokens=256, max_prefill_tokens=16384, block_size=16, seed=0, tp_group=None) -> dict:
    from ..serving.llm_engine import LLMEngine, SamplingParams
    cfg = model.config
    dev = next(model.parameters()).device
    blocks = requests * ((prompt_len + new_tokens + block_size - 1) // block_size) + 64
    eng = LLMEngine(model, num_blocks=blocks, block_size=block_size, max_batch_size=requests,
                    max_prefill_tokens=max_prefill_tokens, enable_prefix_cache=False, tp_group=tp_group)
    g = torch.Generator().manual_seed(seed)
    prompts = [torch.randint(0, cfg.vocab_size, (prompt_len,), generator=g).tolist() for _ in range(requests)]
    sp = SamplingParams(max_new_tokens=new_tokens)
    with torch.no_grad():
        # warm-up: one short request through prefill and a few decode steps (allocations, kernel loading)
        eng.generate([prompts[0][: min(prompt_len, 128)]], SamplingParams(max_new_tokens=4))
        eng.finished.clear()
        eng.stats = {k: 0 for k in eng.stats}
        if dev.type == "cuda":
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        ids = [eng.submit(p, sp) for p in prompts]
        eng.run_until_done()
        if dev.type == "cuda":
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
    done = [eng.finished[i] for i in ids]
    ttft = sorted(r.first_token_time - r.arrival for r in done)
    out_tokens = sum(len(r.output) for r in done)
    pct = lambda q: ttft[min(len(ttft) - 1, int(q * len(ttft)))]  # noqa: E731
    return {"metric": "serving output tokens/sec", "value": out_tokens / dt, "unit": "tokens/s", "requests": requests,
            "prompt_len": prompt_len, "new_tokens": new_tokens, "seconds": dt, "output_tokens": out_tokens,
            "prefill_tokens": eng.stats["prefill_tokens"], "engine_steps": eng.stats["steps"],
            "ttft_p50_s": pct(0.5), "ttft_p95_s": pct(0.95), "ttft_min_s": ttft[0],
            "total_tokens_per_s": (out_tokens + eng.stats["prefill_tokens"]) / dt}


def _engine_kwargs(requests, prompt_len, new_tokens, max_prefill_tokens, block_size, tp_group=None):
    blocks = requests * ((prompt_len + new_tokens + block_size - 1) // block_size) + 64
    kw = dict(num_blocks=blocks, block_size=block_size, max_batch_size=requests, max_prefill_tokens=max_prefill_tokens,
              enable_prefix_cache=False)
    if tp_group is not None:
        kw["tp_group"] = tp_group
    return kw


def _http_clients(port, prompts, new_tokens, warm, conn):
    """Client side of ``run_http`` in a process of its own (threads in the server's process would share its
    interpreter lock with the thread that launches kernels and trickle their requests out over seconds): one thread
    per request, all released together when the parent says go."""
    import http.client
    import threading

    def post(ids, n):
        c = http.client.HTTPConnection("127.0.0.1", port, timeout=3600)
        t0 = time.perf_counter()
        c.request("POST", "/v1/generate", json.dumps({"prompt_token_ids": ids, "max_new_tokens": n}),
                  {"Content-Type": "application/json"})
        resp = c.getresponse()
        body = json.loads(resp.read())
        c.close()
        if resp.status != 200:
            raise RuntimeError(f"HTTP {resp.status}: {body}")
        return body, time.perf_counter() - t0

    try:
        for _ in range(2):                      # warm-up (allocations, kernel loading, graph capture)
            post(warm, 4)
        bodies = [json.dumps({"prompt_token_ids": p, "max_new_tokens": new_tokens}) for p in prompts]
        del bodies
        conn.send("ready")
        conn.recv()                             # go
        results, errors = [None] * len(prompts), []

        def worker(i):
            try:
                body, dt = post(prompts[i], new_tokens)
                results[i] = (body["completion_tokens"], body["ttft_s"], dt)
            except Exception as e:  # noqa: BLE001  (reported after the run)
                errors.append(f"request {i}: {type(e).__name__}: {e}")

        t0 = time.perf_counter()
        threads = [threading.Thread(target=worker, args=(i,)) for i in range(len(prompts))]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        conn.send({"seconds": time.perf_counter() - t0, "results": results, "errors": errors})
    except Exception as e:  # noqa: BLE001
        conn.send({"seconds": 0.0, "results": [], "errors": [f"client process: {type(e).__name__}: {e}"]})


def run_http(model, requests=64, prompt_len=2048, new_tokens=256, max_prefill_tokens=16384, block_size=16, seed=0,
             tp_group=None) -> dict:
    """The workload of ``run`` sent through ``POST /v1/generate`` of the FastAPI front-end (uvicorn, loopback) by a
    client process. With ``tp_group`` this is the leader's side of tensor-parallel serving; the other ranks run
    ``serving.server.tp_follow`` with the same engine arguments."""
    import multiprocessing as mp
    import socket
    import threading

    import uvicorn

    from ..serving.server import create_app
    cfg = model.config
    app = create_app({"bench": {"model": model, "engine_kwargs": _engine_kwargs(
        requests, prompt_len, new_tokens, max_prefill_tokens, block_size, tp_group)}})
    with socket.socket() as sck:
        sck.bind(("127.0.0.1", 0))
        port = sck.getsockname()[1]
    server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="error"))
    th = threading.Thread(target=server.run, daemon=True)
    th.start()
    t_wait = time.perf_counter()
    while not server.started:
        if time.perf_counter() - t_wait > 60:
            raise RuntimeError("HTTP server did not start")
        time.sleep(0.05)
    g = torch.Generator().manual_seed(seed)
    prompts = [torch.randint(0, cfg.vocab_size, (prompt_len,), generator=g).tolist() for _ in range(requests)]
    ctx = mp.get_context("spawn")
    parent, child = ctx.Pipe()
    proc = ctx.Process(target=_http_clients, args=(port, prompts, new_tokens, prompts[0][: min(prompt_len, 128)], child),
                       daemon=True)
    proc.start()
    msg = parent.recv()                          # "ready" after the warm-up requests, or an error record
    if msg != "ready":
        raise RuntimeError(f"HTTP client process failed: {msg}")
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    parent.send("go")
    out = parent.recv()
    proc.join(30)
    server.should_exit = True
    th.join(10)
    for w in app.state.workers.values():
        w.stop()
    if out["errors"]:
        raise RuntimeError(f"{len(out['errors'])} of {requests} requests failed; first: {out['errors'][0]}")
    dt = out["seconds"]
    out_tokens = sum(r[0] for r in out["results"])
    ttft = sorted(r[1] for r in out["results"])
    lat = sorted(r[2] for r in out["results"])
    pct = lambda v, q: v[min(len(v) - 1, int(q * len(v)))]  # noqa: E731
    return {"metric": "serving output tokens/sec", "value": out_tokens / dt, "unit": "tokens/s", "requests": requests,
            "prompt_len": prompt_len, "new_tokens": new_tokens, "seconds": dt, "output_tokens": out_tokens,
            "ttft_p50_s": pct(ttft, 0.5), "ttft_p95_s": pct(ttft, 0.95), "ttft_min_s": ttft[0],
            "latency_p50_s": pct(lat, 0.5), "latency_max_s": lat[-1],
            "front_end": "HTTP POST /v1/generate (FastAPI on uvicorn, loopback; clients in their own process), "
                         "prompts as token ids"}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--quantize", choices=["none", "fp8", "int4"], default="none")
    ap.add_argument("--max-prefill-tokens", type=int, default=16384)
    ap.add_argument("--http", action="store_true",
                    help="send the requests through POST /v1/generate (under torchrun: rank 0 serves, the others mirror)")
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    import os
    from ..models import create_model
    cuda = torch.cuda.is_available()
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    tp_group = None
    if world > 1:   # under torchrun: tensor parallelism over all ranks (every rank runs the same scheduler)
        import torch.distributed as dist
        if cuda:
            torch.cuda.set_device(local)
        dist.init_process_group("nccl" if cuda else "gloo", **({"device_id": dev} if cuda else {}))
        tp_group = dist.group.WORLD
    torch.manual_seed(0)
    spec = a.model
    if spec.endswith(".json"):   # a model configuration file instead of a preset name
        from ..models import ModelConfig
        spec = ModelConfig.from_json(spec)
    model = create_model(spec, dtype=torch.bfloat16 if cuda else torch.float32, device=dev).eval()
    model.config.max_position_embeddings = max(model.config.max_position_embeddings, a.prompt_len + a.new_tokens)
    if a.quantize != "none":
        from ..ops.quant import quantize_model_
        quantize_model_(model, a.quantize)
    if a.http and world > 1 and rank != 0:
        from ..serving.server import tp_follow
        with torch.no_grad():
            tp_follow(model, _engine_kwargs(a.requests, a.prompt_len, a.new_tokens, a.max_prefill_tokens, 16, tp_group))
        r = {}
    elif a.http:
        r = run_http(model, a.requests, a.prompt_len, a.new_tokens, a.max_prefill_tokens, tp_group=tp_group)
    else:
        r = run(model, a.requests, a.prompt_len, a.new_tokens, a.max_prefill_tokens, tp_group=tp_group)
    r["config"] = {"model": a.model, "weights": "bf16" if a.quantize == "none" else a.quantize, "kv_cache": "bf16" if cuda else "fp32",
                   "parallelism": (f"tp{world}" if world > 1 else "1 GPU") if cuda else (f"cpu tp{world}" if world > 1 else "cpu"),
                   "data": "random token ids, random-init weights"}
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        if rank != 0:
            dist.destroy_process_group()
            return 0
    if cuda:
        from ..ops import check_status
        check_status()
    print(json.dumps(r), flush=True)
    if a.out:
        json.dump(r, open(a.out, "w"), indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())

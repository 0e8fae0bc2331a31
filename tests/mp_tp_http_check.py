"""Tensor-parallel serving behind the HTTP front-end on gloo ranks: rank 0 serves ``POST /v1/generate`` (uvicorn,
loopback) through ``TPEngineWorker``, the other ranks mirror it with ``tp_follow``; the tokens that come back over HTTP
must be those of the single-rank engine. ``python mp_tp_http_check.py <world> <port>``."""
import json
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _run(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from sneppx_alg_b200.models import ModelConfig, build_model
    from sneppx_alg_b200.serving.llm_engine import LLMEngine, SamplingParams
    from sneppx_alg_b200.serving.server import create_app, tp_follow
    torch.manual_seed(0)
    cfg = ModelConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=128,
                      vocab_size=160, max_position_embeddings=128, rms_norm_eps=1e-5)
    model = build_model(cfg).eval()
    prompts = [[3, 9, 27, 81, 5], [7, 7], [100, 2, 150, 4, 9, 9, 31, 8, 64], [12]]
    lens = [6, 9, 4, 7]
    kw = dict(num_blocks=64, block_size=4, max_batch_size=2, tp_group=dist.group.WORLD)
    if rank != 0:
        with torch.no_grad():
            tp_follow(model, kw)
    else:
        import http.client
        import socket
        import threading
        import time

        import uvicorn
        ref = LLMEngine(model, num_blocks=64, block_size=4, max_batch_size=2)
        rids = [ref.submit(p, SamplingParams(max_new_tokens=n)) for p, n in zip(prompts, lens)]
        ref.run_until_done()
        want = [ref.finished[i].output for i in rids]
        app = create_app({"m": {"model": model, "engine_kwargs": kw}})
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            hp = s.getsockname()[1]
        server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=hp, log_level="error"))
        th = threading.Thread(target=server.run, daemon=True)
        th.start()
        t0 = time.time()
        while not server.started:
            assert time.time() - t0 < 60
            time.sleep(0.05)
        got = [None] * len(prompts)

        def post(i):
            c = http.client.HTTPConnection("127.0.0.1", hp, timeout=120)
            c.request("POST", "/v1/generate", json.dumps({"prompt_token_ids": prompts[i], "max_new_tokens": lens[i]}),
                      {"Content-Type": "application/json"})
            r = c.getresponse()
            body = json.loads(r.read())
            assert r.status == 200, body
            got[i] = body["token_ids"]

        ts = [threading.Thread(target=post, args=(i,)) for i in range(len(prompts))]
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        server.should_exit = True
        th.join(10)
        for w in app.state.workers.values():
            w.stop()
        assert got == want, (got, want)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    world, port = int(sys.argv[1]), int(sys.argv[2])
    mp.spawn(_run, args=(world, port), nprocs=world, join=True)
    print("TP_HTTP_OK")

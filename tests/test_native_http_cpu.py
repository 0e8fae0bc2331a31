"""C++ HTTP front-end: routing with {param}, Bearer auth, status codes, large responses, counters, concurrency."""
import json
import threading
import urllib.error
import urllib.request

import pytest

from sneppx_alg_b200.serving.native_http import HTTPError, NativeHttpServer, serve_engine


def _req(port, method, path, body=None, token=None):
    r = urllib.request.Request(f"http://127.0.0.1:{port}{path}", data=body, method=method)
    if token:
        r.add_header("Authorization", f"Bearer {token}")
    try:
        with urllib.request.urlopen(r, timeout=10) as resp:
            return resp.status, resp.read()
    except urllib.error.HTTPError as e:
        return e.code, e.read()


class _Engine:
    def generate(self, prompt, max_new_tokens=32, **kw):
        return {"generated_text": prompt[::-1], "completion_tokens": max_new_tokens, "sampling": kw}


def test_rest_surface_auth_and_errors():
    srv = serve_engine(_Engine(), {"llama3-8b": {"params": 8.0e9}}, token="k3y")
    p = srv.port
    try:
        assert _req(p, "GET", "/v1/health") == (200, b'{"status": "ok"}')           # public route
        assert _req(p, "GET", "/v1/models")[0] == 401                                # protected
        assert _req(p, "GET", "/v1/models", token="bad")[0] == 401
        st, body = _req(p, "GET", "/v1/models", token="k3y")
        assert st == 200 and json.loads(body)["models"][0]["id"] == "llama3-8b"
        assert json.loads(_req(p, "GET", "/v1/models/llama3-8b", token="k3y")[1])["params"] == 8.0e9
        assert _req(p, "GET", "/v1/models/none", token="k3y")[0] == 404
        assert _req(p, "GET", "/v1/nothing", token="k3y")[0] == 404
        assert _req(p, "DELETE", "/v1/models", token="k3y")[0] == 405
        st, body = _req(p, "POST", "/v1/generate", json.dumps({"prompt": "abc", "max_new_tokens": 4, "top_k": 5}).encode(), "k3y")
        out = json.loads(body)
        assert st == 200 and out["generated_text"] == "cba" and out["completion_tokens"] == 4 and out["sampling"] == {"top_k": 5}
        assert _req(p, "POST", "/v1/generate", b"not json", "k3y")[0] == 400
        assert _req(p, "POST", "/v1/generate", json.dumps({"prompt": "x", "max_new_tokens": 99999}).encode(), "k3y")[0] == 400
        assert srv.hits("POST", "/v1/generate") == 3
        m = json.loads(_req(p, "GET", "/metrics/native")[1])
        assert m["requests"] >= 11 and m["rejected"] >= 4
    finally:
        srv.stop()


def test_large_bodies_handler_errors_and_concurrency():
    srv = NativeHttpServer(max_body=1 << 16)

    @srv.route("POST", "/echo/{name}/size")
    def echo(params, body):
        return {"name": params["name"], "n": len(body)}

    calls = []

    @srv.route("GET", "/big")
    def big(_p, _b):
        calls.append(1)
        return b"x" * 300000  # larger than the first response buffer: the server asks again with room

    @srv.route("GET", "/boom")
    def boom(_p, _b):
        raise RuntimeError("bug")

    @srv.route("GET", "/teapot")
    def teapot(_p, _b):
        raise HTTPError(403, "no")

    port = srv.start(workers=4)
    try:
        assert json.loads(_req(port, "POST", "/echo/a%20b/size", b"z" * 50000)[1]) == {"name": "a%20b", "n": 50000}
        assert _req(port, "POST", "/echo/a/size", b"z" * 70000)[0] == 413
        st, body = _req(port, "GET", "/big")
        assert st == 200 and len(body) == 300000 and len(calls) == 1  # the handler ran once
        st, body = _req(port, "GET", "/boom")
        assert st == 500 and b"RuntimeError" in body
        assert _req(port, "GET", "/teapot") == (403, b'{"error": "no"}')
        results = []

        def hammer():
            for _ in range(20):
                results.append(_req(port, "POST", "/echo/t/size", b"12345")[0])

        ths = [threading.Thread(target=hammer) for _ in range(8)]
        [t.start() for t in ths]
        [t.join() for t in ths]
        assert results == [200] * 160 and srv.hits("POST", "/echo/{name}/size") == 161
    finally:
        srv.stop()


def test_text_engine_behind_native_front_end():
    import torch
    from sneppx_alg_b200.models import create_model
    from sneppx_alg_b200.serving.native_http import TextEngine
    torch.manual_seed(0)
    model = create_model("llama3-tiny").eval()
    eng = TextEngine(model, model_id="tiny", num_blocks=64, max_batch_size=4)
    srv = serve_engine(eng, {"tiny": {"family": "llama"}})
    try:
        st, body = _req(srv.port, "POST", "/v1/generate", json.dumps({"prompt": "hello", "max_new_tokens": 5}).encode())
        out = json.loads(body)
        assert st == 200 and out["completion_tokens"] == 5 and out["prompt_tokens"] == 5 and out["model"] == "tiny"
        assert len(out["token_ids"]) == 5 and out["total_tokens"] == 10
        # a stop string taken from the middle of a longer greedy continuation ends the request early and is cut off
        long = json.loads(_req(srv.port, "POST", "/v1/generate", json.dumps({"prompt": "hello", "max_new_tokens": 12}).encode())[1])
        text = long["generated_text"]
        stop = text[4:6]
        cut = json.loads(_req(srv.port, "POST", "/v1/generate", json.dumps(
            {"prompt": "hello", "max_new_tokens": 12, "stop_strings": [stop]}).encode())[1])
        assert cut["generated_text"] == text[:text.find(stop)] and cut["completion_tokens"] < 12
    finally:
        srv.stop()
        eng.stop()


def test_serve_cli_native_dry_run(capsys):
    from sneppx_alg_b200.cli import serve_main
    assert serve_main(["--front-end", "native", "--dry-run", "--model-config", "llama3-tiny"]) == 0
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["front_end"] == "native"

"""Circuit breaker, load balancer and the fail-over HTTP client (``utils/client_net.py``) against small in-process
HTTP servers."""
import collections
import http.server
import json
import ssl
import threading

import pytest

from sneppx_alg_b200.utils import client_net as cn


def test_circuit_breaker_states():
    now = [0.0]
    cb = cn.CircuitBreaker("db", failure_threshold=3, recovery_timeout_s=10.0, half_open_max_calls=1, clock=lambda: now[0])
    boom = lambda: 1 / 0            # noqa: E731
    assert cb.call(lambda: 7) == 7 and cb.state == cb.CLOSED
    for _ in range(2):
        with pytest.raises(ZeroDivisionError):
            cb.call(boom)
    assert cb.state == cb.CLOSED and cb.failure_count == 2
    assert cb.call(lambda: 1) == 1 and cb.failure_count == 0            # a success clears the count
    for _ in range(3):
        with pytest.raises(ZeroDivisionError):
            cb.call(boom)
    assert cb.state == cb.OPEN
    with pytest.raises(cn.CircuitOpenError):
        cb.call(lambda: 1)                                                  # fails fast, the function is not called
    assert cb.rejected == 1
    now[0] = 10.0
    assert cb.state == cb.HALF_OPEN
    with pytest.raises(ZeroDivisionError):
        cb.call(boom)                                                       # the probe fails: open again, timer restarts
    assert cb.state == cb.OPEN
    now[0] = 19.0
    assert cb.state == cb.OPEN
    now[0] = 20.0
    assert cb.call(lambda: "ok") == "ok" and cb.state == cb.CLOSED
    cb.record_failure()
    cb.reset()
    assert cb.failure_count == 0 and cb.state == cb.CLOSED


def test_load_balancer_strategies():
    rr = cn.LoadBalancer("round_robin")
    for p in (1, 2, 3):
        rr.add_backend("h", p)
    assert [rr.next_backend().port for _ in range(6)] == [1, 2, 3, 1, 2, 3]
    assert rr.mark_unhealthy("h", 2) and not rr.mark_unhealthy("h", 9)
    assert {rr.next_backend().port for _ in range(6)} == {1, 3}
    rr.mark_healthy("h", 2)
    assert rr.remove_backend("h", 1) and not rr.remove_backend("h", 1) and len(rr.healthy_backends()) == 2
    w = cn.LoadBalancer("weighted")
    w.add_backend("a", 1, weight=5)
    w.add_backend("b", 1, weight=1)
    w.add_backend("c", 1, weight=1)
    picks = [w.next_backend().host for _ in range(70)]
    assert collections.Counter(picks) == {"a": 50, "b": 10, "c": 10} and picks[:7].count("a") == 5 and "aaaaa" not in "".join(picks[:7])
    lc = cn.LoadBalancer("least_conn")
    lc.add_backend("x", 1)
    lc.add_backend("y", 1)
    first, second = lc.acquire(), lc.acquire()
    assert {first.host, second.host} == {"x", "y"}
    lc.release(first)
    assert lc.acquire().host == first.host                                  # the one with fewer requests in flight
    rnd = cn.LoadBalancer("random", seed=0)
    rnd.add_backend("p", 1)
    rnd.add_backend("q", 1)
    assert {rnd.next_backend().host for _ in range(40)} == {"p", "q"}
    rnd.mark_unhealthy("p", 1)
    rnd.mark_unhealthy("q", 1)
    assert rnd.next_backend() is None
    with pytest.raises(ValueError):
        cn.LoadBalancer("fastest")
    with pytest.raises(ValueError):
        w.add_backend("d", 1, weight=0)


def _server(name, fail=False):
    hits = []

    class H(http.server.BaseHTTPRequestHandler):
        def _reply(self):
            n = int(self.headers.get("Content-Length") or 0)
            body = self.rfile.read(n) if n else b""
            hits.append((self.command, self.path, body))
            code = 503 if fail else (404 if self.path == "/missing" else 200)
            out = json.dumps({"server": name, "method": self.command, "echo": body.decode()}).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(out)))
            self.end_headers()
            self.wfile.write(out)

        do_GET = do_POST = do_PUT = do_DELETE = _reply

        def log_message(self, *a):
            pass

    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    return srv, hits


def test_http_client_verbs_failover_and_breaker():
    good, good_hits = _server("good")
    bad, bad_hits = _server("bad", fail=True)
    try:
        c = cn.HttpClient(f"http://127.0.0.1:{good.server_port}/", timeout_s=5.0, headers={"X-Test": "1"})
        r = c.post("/v1/echo", {"a": 1})
        assert r.ok and r.json() == {"server": "good", "method": "POST", "echo": '{"a": 1}'} and good_hits[-1][1] == "/v1/echo"
        assert c.put("x", b"raw").json()["echo"] == "raw" and c.delete("/x").json()["method"] == "DELETE"
        missing = c.get("/missing")
        assert missing.status == 404 and not missing.ok                      # error statuses are returned, not raised
        lb = cn.LoadBalancer("round_robin")
        lb.add_backend("127.0.0.1", bad.server_port)
        lb.add_backend("127.0.0.1", 1)                                       # nothing listens there
        lb.add_backend("127.0.0.1", good.server_port)
        fc = cn.HttpClient(balancer=lb, retries=2, timeout_s=2.0)
        assert fc.get("/health").json()["server"] == "good"                  # went past the back-end that answers 503
        assert bad.server_port not in [b.port for b in lb.healthy_backends()] and len(bad_hits) == 1
        assert all(fc.get("/again").json()["server"] == "good" for _ in range(3))     # and past the refused connection
        assert [b.port for b in lb.healthy_backends()] == [good.server_port]
        lb.mark_unhealthy("127.0.0.1", good.server_port)
        with pytest.raises(ConnectionError):
            fc.get("/health")
        now = [0.0]
        cb = cn.CircuitBreaker(failure_threshold=2, recovery_timeout_s=5.0, clock=lambda: now[0])
        guarded = cn.HttpClient(balancer=lb, breaker=cb, retries=0)
        for _ in range(2):
            with pytest.raises(ConnectionError):
                guarded.get("/health")
        with pytest.raises(cn.CircuitOpenError):
            guarded.get("/health")
        lb.mark_healthy("127.0.0.1", good.server_port)
        now[0] = 5.0
        assert guarded.get("/health").ok and cb.state == cb.CLOSED
        with pytest.raises(ValueError):
            cn.HttpClient()
    finally:
        good.shutdown()
        bad.shutdown()


def test_tls_contexts_have_a_modern_floor():
    ctx = cn.tls_client_context()
    assert ctx.minimum_version == ssl.TLSVersion.TLSv1_2 and ctx.verify_mode == ssl.CERT_REQUIRED and ctx.check_hostname
    assert ctx.options & ssl.OP_NO_COMPRESSION
    with pytest.raises((FileNotFoundError, ssl.SSLError, OSError)):
        cn.tls_server_context("/nonexistent/cert.pem", "/nonexistent/key.pem")

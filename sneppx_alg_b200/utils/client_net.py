"""Client-side networking pieces: a circuit breaker, a load balancer over back-ends with health marks, an HTTP client
that uses both, and TLS contexts with modern defaults.

Reference counterparts: ``include/neural_core/network/circuit_breaker.h`` (closed / open / half-open with a failure
threshold, a recovery time-out and a cap on half-open probes), ``load_balancer.h`` (round robin, least connections,
random, weighted; healthy / unhealthy marks), ``http_client.h`` (GET / POST / PUT / DELETE against a base URL with a
time-out) and ``tls_transport.h``. The C++ serving core has its own breaker for the request path
(``csrc/host/serving_core.cpp``); this one wraps arbitrary Python callables.
"""
from __future__ import annotations

import json
import random
import ssl
import threading
import time
import urllib.error
import urllib.request
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple


class CircuitOpenError(RuntimeError):
    pass


class CircuitBreaker:
    """Stops calling a failing dependency for a while. CLOSED: calls pass, consecutive failures are counted; at
    ``failure_threshold`` the breaker OPENs and calls fail fast with ``CircuitOpenError``; after ``recovery_timeout_s``
    it is HALF_OPEN and lets up to ``half_open_max_calls`` probes through: one success closes it, one failure opens
    it again."""

    CLOSED, OPEN, HALF_OPEN = "closed", "open", "half_open"

    def __init__(self, name: str = "", failure_threshold: int = 5, recovery_timeout_s: float = 30.0, half_open_max_calls: int = 1,
                 clock: Callable[[], float] = time.monotonic):
        self.name, self.failure_threshold, self.recovery_timeout_s, self.half_open_max_calls, self.clock = \
            name, failure_threshold, recovery_timeout_s, half_open_max_calls, clock
        self._lock = threading.Lock()
        self.reset()

    def reset(self) -> None:
        self._state, self._failures, self._opened_at, self._probes = self.CLOSED, 0, 0.0, 0
        self.rejected = 0

    @property
    def state(self) -> str:
        with self._lock:
            if self._state == self.OPEN and self.clock() - self._opened_at >= self.recovery_timeout_s:
                self._state, self._probes = self.HALF_OPEN, 0
            return self._state

    @property
    def failure_count(self) -> int:
        return self._failures

    def _admit(self) -> None:
        st = self.state
        with self._lock:
            if st == self.OPEN or (st == self.HALF_OPEN and self._probes >= self.half_open_max_calls):
                self.rejected += 1
                raise CircuitOpenError(f"circuit {self.name or 'breaker'} is {st}")
            if st == self.HALF_OPEN:
                self._probes += 1

    def record_success(self) -> None:
        with self._lock:
            self._state, self._failures = self.CLOSED, 0

    def record_failure(self) -> None:
        with self._lock:
            self._failures += 1
            if self._state == self.HALF_OPEN or self._failures >= self.failure_threshold:
                self._state, self._opened_at = self.OPEN, self.clock()

    def call(self, fn: Callable, *args, **kwargs):
        self._admit()
        try:
            out = fn(*args, **kwargs)
        except Exception:
            self.record_failure()
            raise
        self.record_success()
        return out


@dataclass
class Backend:
    host: str
    port: int
    weight: int = 1
    healthy: bool = True
    active: int = 0                 # requests in flight (least-connections)
    served: int = 0
    _credit: float = field(default=0.0, repr=False)

    @property
    def address(self) -> Tuple[str, int]:
        return self.host, self.port


class LoadBalancer:
    """Picks a healthy back-end by ``round_robin``, ``least_conn``, ``random`` or ``weighted`` (smooth weighted round
    robin: over any window the picks follow the weights and are as evenly interleaved as possible)."""

    STRATEGIES = ("round_robin", "least_conn", "random", "weighted")

    def __init__(self, strategy: str = "round_robin", seed: Optional[int] = None):
        if strategy not in self.STRATEGIES:
            raise ValueError(f"unknown strategy {strategy!r}")
        self.strategy, self.backends, self._next = strategy, [], 0
        self._rng = random.Random(seed)
        self._lock = threading.Lock()

    def _find(self, host: str, port: int) -> Optional[Backend]:
        return next((b for b in self.backends if b.address == (host, port)), None)

    def add_backend(self, host: str, port: int, weight: int = 1) -> Backend:
        if weight < 1:
            raise ValueError("weight must be at least 1")
        with self._lock:
            b = self._find(host, port)
            if b is None:
                b = Backend(host, port, weight)
                self.backends.append(b)
            else:
                b.weight = weight
            return b

    def remove_backend(self, host: str, port: int) -> bool:
        with self._lock:
            b = self._find(host, port)
            if b is None:
                return False
            self.backends.remove(b)
            return True

    def mark_unhealthy(self, host: str, port: int) -> bool:
        b = self._find(host, port)
        if b is not None:
            b.healthy = False
        return b is not None

    def mark_healthy(self, host: str, port: int) -> bool:
        b = self._find(host, port)
        if b is not None:
            b.healthy = True
        return b is not None

    def healthy_backends(self) -> List[Backend]:
        return [b for b in self.backends if b.healthy]

    def next_backend(self) -> Optional[Backend]:
        with self._lock:
            live = self.healthy_backends()
            if not live:
                return None
            if self.strategy == "round_robin":
                b = live[self._next % len(live)]
                self._next += 1
            elif self.strategy == "least_conn":
                b = min(live, key=lambda x: (x.active, x.served))
            elif self.strategy == "random":
                b = self._rng.choice(live)
            else:
                total = sum(x.weight for x in live)
                for x in live:
                    x._credit += x.weight
                b = max(live, key=lambda x: x._credit)
                b._credit -= total
            b.served += 1
            return b

    def acquire(self) -> Optional[Backend]:
        b = self.next_backend()
        if b is not None:
            b.active += 1
        return b

    def release(self, backend: Backend) -> None:
        backend.active = max(0, backend.active - 1)


@dataclass
class HttpResponse:
    status: int
    body: bytes
    headers: Dict[str, str]

    def json(self) -> Any:
        return json.loads(self.body)

    @property
    def ok(self) -> bool:
        return 200 <= self.status < 300


class HttpClient:
    """GET / POST / PUT / DELETE against one base URL, or, with a ``LoadBalancer``, against its healthy back-ends with
    fail-over: a back-end that refuses the connection or answers 5xx is marked unhealthy and the request goes to the
    next one (at most ``retries`` extra attempts). An optional ``CircuitBreaker`` guards the whole client. HTTP error
    statuses are returned, not raised; only transport failures raise."""

    def __init__(self, base_url: Optional[str] = None, timeout_s: float = 5.0, balancer: Optional[LoadBalancer] = None,
                 breaker: Optional[CircuitBreaker] = None, retries: int = 2, headers: Optional[Dict[str, str]] = None,
                 scheme: str = "http", context: Optional[ssl.SSLContext] = None):
        if (base_url is None) == (balancer is None):
            raise ValueError("give either a base URL or a load balancer")
        self.base_url, self.timeout_s, self.balancer, self.breaker, self.retries = \
            (base_url.rstrip("/") if base_url else None), timeout_s, balancer, breaker, retries
        self.headers, self.scheme, self.context = dict(headers or {}), scheme, context

    def _once(self, base: str, method: str, path: str, body: Optional[bytes], headers: Dict[str, str]) -> HttpResponse:
        req = urllib.request.Request(base + path, data=body, method=method, headers={**self.headers, **headers})
        try:
            with urllib.request.urlopen(req, timeout=self.timeout_s, context=self.context) as r:
                return HttpResponse(r.status, r.read(), dict(r.headers))
        except urllib.error.HTTPError as e:
            return HttpResponse(e.code, e.read(), dict(e.headers))

    def _send(self, method: str, path: str, body: Optional[bytes], headers: Dict[str, str]) -> HttpResponse:
        if self.balancer is None:
            return self._once(self.base_url, method, path, body, headers)
        last: Optional[Exception] = None
        for _ in range(self.retries + 1):
            b = self.balancer.acquire()
            if b is None:
                break
            try:
                resp = self._once(f"{self.scheme}://{b.host}:{b.port}", method, path, body, headers)
            except (urllib.error.URLError, OSError, TimeoutError) as e:
                self.balancer.mark_unhealthy(b.host, b.port)
                last = e
                continue
            finally:
                self.balancer.release(b)
            if resp.status >= 500:
                self.balancer.mark_unhealthy(b.host, b.port)
                last = RuntimeError(f"{b.host}:{b.port} answered {resp.status}")
                continue
            return resp
        raise ConnectionError(f"no healthy back-end answered ({last})")

    def request(self, method: str, path: str, body=None, headers: Optional[Dict[str, str]] = None) -> HttpResponse:
        headers = dict(headers or {})
        if body is not None and not isinstance(body, (bytes, bytearray)):
            body = json.dumps(body).encode()
            headers.setdefault("Content-Type", "application/json")
        send = lambda: self._send(method, path if path.startswith("/") else "/" + path, body, headers)     # noqa: E731
        return self.breaker.call(send) if self.breaker is not None else send()

    def get(self, path: str, **kw) -> HttpResponse:
        return self.request("GET", path, **kw)

    def post(self, path: str, body=None, **kw) -> HttpResponse:
        return self.request("POST", path, body, **kw)

    def put(self, path: str, body=None, **kw) -> HttpResponse:
        return self.request("PUT", path, body, **kw)

    def delete(self, path: str, **kw) -> HttpResponse:
        return self.request("DELETE", path, **kw)


def tls_client_context(ca_file: Optional[str] = None, certfile: Optional[str] = None, keyfile: Optional[str] = None,
                       check_hostname: bool = True) -> ssl.SSLContext:
    """Client context: TLS 1.2 or newer, certificate verification on, no compression; ``certfile`` / ``keyfile`` add a
    client certificate for mutual TLS."""
    ctx = ssl.create_default_context(cafile=ca_file)
    ctx.minimum_version = ssl.TLSVersion.TLSv1_2
    ctx.options |= ssl.OP_NO_COMPRESSION
    ctx.check_hostname = check_hostname
    if certfile:
        ctx.load_cert_chain(certfile, keyfile)
    return ctx


def tls_server_context(certfile: str, keyfile: str, client_ca: Optional[str] = None) -> ssl.SSLContext:
    """Server context with the same floor; ``client_ca`` turns on mutual TLS (clients must present a certificate it
    signed)."""
    ctx = ssl.SSLContext(ssl.PROTOCOL_TLS_SERVER)
    ctx.minimum_version = ssl.TLSVersion.TLSv1_2
    ctx.options |= ssl.OP_NO_COMPRESSION
    ctx.load_cert_chain(certfile, keyfile)
    if client_ca:
        ctx.verify_mode = ssl.CERT_REQUIRED
        ctx.load_verify_locations(client_ca)
    return ctx

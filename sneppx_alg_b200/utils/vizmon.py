"""vizmon — metrics / timeline store with a small embedded HTTP JSON endpoint (the reference's ``net/http/vizmon.c``
and Python ``vizmon.py``): scalars, histograms and timeline spans, served at ``/metrics.json`` and ``/timeline.json``
for a dashboard; no external dependencies."""
from __future__ import annotations

import json
import threading
import time
from collections import defaultdict, deque
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Dict


class VizMon:
    def __init__(self, history=1024):
        self.scalars: Dict[str, deque] = defaultdict(lambda: deque(maxlen=history))
        self.spans: deque = deque(maxlen=history)
        self.lock = threading.Lock()
        self._srv = None

    def scalar(self, name, value, step=None):
        with self.lock:
            self.scalars[name].append((step if step is not None else len(self.scalars[name]), float(value), time.time()))

    def span(self, name):
        mon = self

        class _Span:
            def __enter__(self):
                self.t0 = time.time()

            def __exit__(self, *exc):
                with mon.lock:
                    mon.spans.append({"name": name, "start": self.t0, "end": time.time()})
        return _Span()

    def histogram(self, name, bins=10):
        vals = [v for _, v, _ in self.scalars.get(name, [])]
        if not vals:
            return {"edges": [], "counts": []}
        lo, hi = min(vals), max(vals)
        w = (hi - lo) / bins or 1.0
        counts = [0] * bins
        for v in vals:
            counts[min(bins - 1, int((v - lo) / w))] += 1
        return {"edges": [lo + i * w for i in range(bins + 1)], "counts": counts}

    def snapshot(self):
        with self.lock:
            return {"scalars": {k: list(v) for k, v in self.scalars.items()}, "spans": list(self.spans)}

    def serve(self, host="127.0.0.1", port=0):
        mon = self

        class H(BaseHTTPRequestHandler):
            def log_message(self, *a):
                pass

            def do_GET(self):
                snap = mon.snapshot()
                body = {"/metrics.json": snap["scalars"], "/timeline.json": snap["spans"]}.get(self.path)
                if body is None:
                    self.send_response(404)
                    self.end_headers()
                    return
                data = json.dumps(body).encode()
                self.send_response(200)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(data)))
                self.end_headers()
                self.wfile.write(data)
        self._srv = ThreadingHTTPServer((host, port), H)
        threading.Thread(target=self._srv.serve_forever, daemon=True).start()
        return self._srv.server_address[1]

    def stop(self):
        if self._srv:
            self._srv.shutdown()
            self._srv = None

"""vizmon — metrics / graph / timeline store with an embedded HTTP dashboard (the reference's ``net/http/vizmon.c``
and Python ``vizmon.py``): scalars, histograms, timeline spans and a model graph, served as JSON at ``/metrics.json``,
``/timeline.json``, ``/graph.json`` and as a page at ``/`` that follows a live WebSocket feed (``/ws``: one JSON text
frame per tick with the samples and spans recorded since the previous one) and falls back to polling. Scalars and
spans live in the native store (``csrc/host/vizmon_store.cpp``: rings, summaries, incremental snapshots by sequence
number); no external dependencies."""
from __future__ import annotations

import json
import threading
import time
from collections import defaultdict, deque
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Dict


def _L():
    import ctypes as C

    from .. import _build
    L = _build.load_host()
    if not getattr(L, "_viz_ready", False):
        L.sx_viz_create.restype = C.c_void_p
        L.sx_viz_create.argtypes = [C.c_size_t]
        L.sx_viz_destroy.argtypes = [C.c_void_p]
        L.sx_viz_scalar.argtypes = [C.c_void_p, C.c_char_p, C.c_longlong, C.c_double, C.c_double]
        L.sx_viz_scalar.restype = C.c_ulonglong
        L.sx_viz_span.argtypes = [C.c_void_p, C.c_char_p, C.c_double, C.c_double]
        L.sx_viz_span.restype = C.c_ulonglong
        L.sx_viz_sequence.argtypes = [C.c_void_p]
        L.sx_viz_sequence.restype = C.c_ulonglong
        L.sx_viz_summary.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p]
        L.sx_viz_snapshot.argtypes = [C.c_void_p, C.c_ulonglong, C.c_char_p, C.c_size_t]
        L.sx_viz_snapshot.restype = C.c_longlong
        L._viz_ready = True
    return L


class VizMon:
    def __init__(self, history=1024):
        self.scalars: Dict[str, deque] = defaultdict(lambda: deque(maxlen=history))
        self.spans: deque = deque(maxlen=history)
        self.lock = threading.Lock()
        self._srv = None
        self.graph_nodes, self.graph_edges = [], []
        self._store = _L().sx_viz_create(history)
        self.ws_clients = 0

    def summary(self, name: str):
        """count / total / min / max / mean / last / p50 / p95 of a series' retained window (native store)."""
        import ctypes as C
        out = (C.c_double * 8)()
        if not _L().sx_viz_summary(self._store, name.encode(), out):
            return None
        keys = ("count", "total", "min", "max", "mean", "last", "p50", "p95")
        return dict(zip(keys, (float(v) for v in out)))

    def updates_since(self, seq: int = 0) -> dict:
        """Samples and spans recorded after sequence number ``seq`` (0: everything retained), plus the new ``seq``."""
        import ctypes as C
        cap = 1 << 16
        while True:
            buf = C.create_string_buffer(cap)
            n = _L().sx_viz_snapshot(self._store, seq, buf, cap)
            if n >= 0:
                return json.loads(buf.value.decode())
            cap = -n + 16

    def set_graph(self, nodes, edges):
        """nodes: [{"id", "label", ...}], edges: [(src id, dst id)]."""
        with self.lock:
            self.graph_nodes, self.graph_edges = list(nodes), [list(e) for e in edges]

    def graph_from_module(self, module, max_depth: int = 2):
        """Module tree of a ``torch.nn.Module`` down to `max_depth` as the dashboard graph."""
        nodes, edges = [{"id": "", "label": type(module).__name__}], []
        for name, m in module.named_modules():
            if name and name.count(".") < max_depth:
                nodes.append({"id": name, "label": f"{name.split('.')[-1]}: {type(m).__name__}",
                              "params": sum(p.numel() for p in m.parameters(recurse=False))})
                edges.append((name.rsplit(".", 1)[0] if "." in name else "", name))
        self.set_graph(nodes, edges)

    def scalar(self, name, value, step=None):
        now = time.time()
        with self.lock:
            self.scalars[name].append((step if step is not None else len(self.scalars[name]), float(value), now))
        _L().sx_viz_scalar(self._store, name.encode(), -1 if step is None else int(step), float(value), now)

    def span(self, name):
        mon = self

        class _Span:
            def __enter__(self):
                self.t0 = time.time()

            def __exit__(self, *exc):
                t1 = time.time()
                with mon.lock:
                    mon.spans.append({"name": name, "start": self.t0, "end": t1})
                _L().sx_viz_span(mon._store, name.encode(), self.t0, t1)
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

    def serve(self, host="127.0.0.1", port=0, ws_interval=0.5):
        mon = self
        from .net import ws_accept_key, ws_encode

        class H(BaseHTTPRequestHandler):
            def log_message(self, *a):
                pass

            def do_GET(self):
                if self.path == "/ws":
                    key = self.headers.get("Sec-WebSocket-Key")
                    if self.headers.get("Upgrade", "").lower() != "websocket" or not key:
                        self.send_response(400)
                        self.end_headers()
                        return
                    self.send_response(101, "Switching Protocols")
                    self.send_header("Upgrade", "websocket")
                    self.send_header("Connection", "Upgrade")
                    self.send_header("Sec-WebSocket-Accept", ws_accept_key(key))
                    self.end_headers()
                    mon.ws_clients += 1
                    seq = 0
                    try:      # the live feed: everything retained first, then only what is new each tick
                        while mon._srv is not None:
                            upd = mon.updates_since(seq)
                            if upd["seq"] != seq or seq == 0:
                                seq = upd["seq"]
                                self.wfile.write(ws_encode(json.dumps(upd).encode(), opcode=1))
                                self.wfile.flush()
                            time.sleep(ws_interval)
                    except (BrokenPipeError, ConnectionError, OSError):
                        pass
                    finally:
                        mon.ws_clients -= 1
                    return
                snap = mon.snapshot()
                if self.path in ("/", "/index.html"):
                    page = _PAGE.encode()
                    self.send_response(200)
                    self.send_header("Content-Type", "text/html; charset=utf-8")
                    self.send_header("Content-Length", str(len(page)))
                    self.end_headers()
                    self.wfile.write(page)
                    return
                body = {"/metrics.json": snap["scalars"], "/timeline.json": snap["spans"],
                        "/graph.json": {"nodes": mon.graph_nodes, "edges": mon.graph_edges}}.get(self.path)
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
            srv, self._srv = self._srv, None
            srv.shutdown()


_PAGE = """<!doctype html><html><head><meta charset="utf-8"><title>sneppx vizmon</title>
<style>body{font:13px monospace;margin:16px;background:#111;color:#ddd}svg{background:#1b1b1b;margin:4px 0}
h3{margin:12px 0 2px}.s{color:#8c8}</style></head><body><h2>sneppx vizmon</h2><div id="m"></div><h3>timeline</h3>
<div id="t"></div><h3>graph</h3><pre id="g"></pre><script>
function spark(v){const w=420,h=48;if(!v.length)return"";const ys=v.map(p=>p[1]),lo=Math.min(...ys),hi=Math.max(...ys);
const pts=v.map((p,i)=>(i*(w-4)/Math.max(v.length-1,1)+2)+","+(h-2-(hi>lo?(p[1]-lo)/(hi-lo):.5)*(h-4))).join(" ");
return`<svg width="${w}" height="${h}"><polyline fill="none" stroke="#6cf" points="${pts}"/></svg>`}
async function tick(){const m=await(await fetch("/metrics.json")).json();let s="";
for(const k in m){const v=m[k];s+=`<h3>${k} <span class=s>${v.length?v[v.length-1][1].toPrecision(5):""}</span></h3>`+spark(v)}
document.getElementById("m").innerHTML=s;const t=await(await fetch("/timeline.json")).json();
document.getElementById("t").innerHTML=t.slice(-12).map(x=>`${x.name}: ${((x.end-x.start)*1e3).toFixed(2)} ms`).join("<br>");
const g=await(await fetch("/graph.json")).json();document.getElementById("g").textContent=g.nodes.map(n=>n.id.split(".").map(_=>"  ").join("")+n.label).join("\n")}
let M={};function draw(){let s="";for(const k in M){const v=M[k];s+=`<h3>${k} <span class=s>${v.length?v[v.length-1][1].toPrecision(5):""}</span></h3>`+spark(v)}
document.getElementById("m").innerHTML=s}
tick();let poll=setInterval(tick,2000);try{const ws=new WebSocket((location.protocol=="https:"?"wss://":"ws://")+location.host+"/ws");
ws.onopen=()=>clearInterval(poll);ws.onmessage=e=>{const u=JSON.parse(e.data);for(const k in u.scalars){M[k]=(M[k]||[]).concat(u.scalars[k]).slice(-1024)}draw();
if(u.spans.length)document.getElementById("t").innerHTML=u.spans.slice(-12).map(x=>`${x.name}: ${((x.end-x.start)*1e3).toFixed(2)} ms`).join("<br>")};
ws.onclose=()=>{poll=setInterval(tick,2000)}}catch(e){}</script></body></html>"""

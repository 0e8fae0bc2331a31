"""vizmon — metrics / graph / timeline store with an embedded HTTP dashboard (the reference's ``net/http/vizmon.c``
and Python ``vizmon.py``): scalars, histograms, timeline spans and a model graph, served as JSON at ``/metrics.json``,
``/timeline.json``, ``/graph.json`` and as a self-refreshing page at ``/``; no external dependencies."""
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
        self.graph_nodes, self.graph_edges = [], []

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
            self._srv.shutdown()
            self._srv = None


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
tick();setInterval(tick,2000)</script></body></html>"""

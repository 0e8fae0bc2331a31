"""The reference's tensor micro-benchmark list (``tests/benchmark/bench_tensor.c``, published in
``benchmarks/baseline.json``) on this framework's tensors, and a regression checker with the reference's thresholds
(``tests/README.md:248-253``: GEMM 10 %, autodiff 15 %, allocator 5 %, algorithms 10 %).

``python -m sneppx_alg_b200.benchmarks.tensor_ops [--device cpu|cuda] [--out file.json]``
``python -m sneppx_alg_b200.benchmarks.tensor_ops --compare old.json new.json``

Each op is timed like the reference does it: mean / min / max over N runs of one call (fp32, same shapes). On CUDA a
run is bracketed by device synchronisation, so small ops measure launch latency. ``published_ms`` is the reference's
figure (unstated CPU, its author's development machine); ``vs_published`` = published / ours, above 1 is faster.
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import torch

# (name, published mean ms, runs, category) in the order of the reference's output
PUBLISHED = [
    ("create [16,16]", 0.001, 2000, "allocator"), ("create [256,256]", 0.158, 1000, "allocator"),
    ("create [1024,1024]", 4.871, 100, "allocator"), ("fill_f32 [256,256]", 0.039, 1000, "algorithms"),
    ("fill_f32 [1024,1024]", 0.979, 100, "algorithms"), ("add [256,256]", 0.200, 1000, "algorithms"),
    ("mul [256,256]", 0.206, 1000, "algorithms"), ("matmul [128,128]x[128,128]", 3.236, 500, "gemm"),
    ("matmul [64,256]x[256,64]", 1.552, 500, "gemm"), ("slice dim0 0:64 [128,128]", 0.0005, 1000, "algorithms"),
    ("reshape [16384]", 0.0005, 1000, "algorithms"), ("transpose 0,1 [128,128]", 0.001, 1000, "algorithms"),
    ("relu [256,256]", 0.343, 500, "algorithms"), ("sigmoid [256,256]", 1.334, 500, "algorithms"),
    ("softmax dim=1 [256,256]", 1.378, 500, "algorithms"), ("sqrt [256,256]", 0.606, 500, "algorithms"),
    ("sum dim=0 [256,256]", 0.061, 500, "algorithms"), ("mean dim=1 [256,256]", 0.273, 500, "algorithms"),
    ("matmul backward [128,128]x[128,128]", None, 200, "autodiff"),
]
THRESHOLDS = {"gemm": 0.10, "autodiff": 0.15, "allocator": 0.05, "algorithms": 0.10}


def _ops(dev):
    r = lambda *s: torch.rand(*s, device=dev)  # noqa: E731
    a256, b256, p256 = r(256, 256), r(256, 256), r(256, 256) + 0.5
    a128, b128 = r(128, 128), r(128, 128)
    a64, b64 = r(64, 256), r(256, 64)
    f256, f1024 = torch.empty(256, 256, device=dev), torch.empty(1024, 1024, device=dev)
    ga, gb = r(128, 128).requires_grad_(True), r(128, 128).requires_grad_(True)

    def mm_bwd():
        ga.grad = gb.grad = None
        (ga @ gb).sum().backward()

    return {
        "create [16,16]": lambda: torch.zeros(16, 16, device=dev), "create [256,256]": lambda: torch.zeros(256, 256, device=dev),
        "create [1024,1024]": lambda: torch.zeros(1024, 1024, device=dev), "fill_f32 [256,256]": lambda: f256.fill_(1.5),
        "fill_f32 [1024,1024]": lambda: f1024.fill_(1.5), "add [256,256]": lambda: a256 + b256, "mul [256,256]": lambda: a256 * b256,
        "matmul [128,128]x[128,128]": lambda: a128 @ b128, "matmul [64,256]x[256,64]": lambda: a64 @ b64,
        "slice dim0 0:64 [128,128]": lambda: a128[0:64], "reshape [16384]": lambda: a128.reshape(16384),
        "transpose 0,1 [128,128]": lambda: a128.transpose(0, 1), "relu [256,256]": lambda: torch.relu(a256),
        "sigmoid [256,256]": lambda: torch.sigmoid(a256), "softmax dim=1 [256,256]": lambda: torch.softmax(a256, dim=1),
        "sqrt [256,256]": lambda: torch.sqrt(p256), "sum dim=0 [256,256]": lambda: a256.sum(dim=0),
        "mean dim=1 [256,256]": lambda: a256.mean(dim=1), "matmul backward [128,128]x[128,128]": mm_bwd,
    }


def run(device="cpu", scale_runs=1.0):
    dev = torch.device(device)
    ops = _ops(dev)
    sync = torch.cuda.synchronize if dev.type == "cuda" else (lambda: None)
    rows = []
    for name, published, runs, cat in PUBLISHED:
        fn = ops[name]
        for _ in range(5):
            fn()
        sync()
        ts = []
        for _ in range(max(10, int(runs * scale_runs))):
            t0 = time.perf_counter()
            fn()
            sync()
            ts.append((time.perf_counter() - t0) * 1e3)
        mean = sum(ts) / len(ts)
        rows.append({"op": name, "category": cat, "mean_ms": mean, "min_ms": min(ts), "max_ms": max(ts), "runs": len(ts),
                     "published_ms": published, "vs_published": (published / mean) if published else None})
    return {"device": str(dev), "threads": torch.get_num_threads(), "dtype": "fp32", "results": rows}


def compare(old: dict, new: dict, thresholds=None):
    """Regressions: ops whose min time grew by more than their category's threshold. Returns (ok, report rows)."""
    th = dict(THRESHOLDS, **(thresholds or {}))
    before = {r["op"]: r for r in old["results"]}
    rows, ok = [], True
    for r in new["results"]:
        b = before.get(r["op"])
        if b is None:
            continue
        change = r["min_ms"] / max(b["min_ms"], 1e-9) - 1.0
        bad = change > th[r["category"]]
        ok &= not bad
        rows.append({"op": r["op"], "category": r["category"], "change": change, "limit": th[r["category"]], "regressed": bad})
    return ok, rows


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--out", default=None)
    ap.add_argument("--compare", nargs=2, metavar=("OLD", "NEW"))
    a = ap.parse_args(argv)
    if a.compare:
        ok, rows = compare(json.load(open(a.compare[0])), json.load(open(a.compare[1])))
        for r in rows:
            print(f"{'REGRESSED' if r['regressed'] else 'ok       '} {r['op']:40s} {100 * r['change']:+7.1f} %  (limit {100 * r['limit']:.0f} %)")
        return 0 if ok else 1
    res = run(a.device)
    for r in res["results"]:
        vs = f"{r['vs_published']:8.1f} x" if r["vs_published"] else "       -"
        print(f"{r['op']:40s} {r['mean_ms']:9.4f} ms  (min {r['min_ms']:8.4f}  max {r['max_ms']:8.4f}  runs {r['runs']})  vs published {vs}")
    if a.out:
        json.dump(res, open(a.out, "w"), indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())

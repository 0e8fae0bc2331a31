"""Performance regression gate: compares the results of the kernel benchmarks with stored floors.

    python -m sneppx_alg_b200.benchmarks.kernels all --out results.json
    python -m sneppx_alg_b200.benchmarks.regression results.json            # exit code 1 when a kernel fell below its floor

The floors (``thresholds.json`` beside this file) are 85 % of the roofline fractions measured on a B200, so ordinary
run-to-run variation passes and a real slow-down does not. ``--update`` rewrites the floors from a results file
(at ``--margin`` of the new values) after an intended change. The reference documents thresholds of this kind for its
C micro-benchmarks (tests/README.md:248-253); this is the executable form for the GPU kernels.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict, List, Tuple

HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT = os.path.join(HERE, "thresholds.json")


def load_thresholds(path: str = DEFAULT) -> Dict[str, dict]:
    with open(path) as f:
        return {k: v for k, v in json.load(f).items() if not k.startswith("_")}


def compare(results: List[dict], thresholds: Dict[str, dict]) -> Tuple[List[dict], List[str]]:
    """(one row per thresholded case, names of cases that have a floor but no result). A row: case, metric, value,
    floor, ok. Only full-size results count (``small`` results are profiler-sized)."""
    by_case = {r["case"]: r for r in results if not r.get("small")}
    rows, missing = [], []
    for case, t in sorted(thresholds.items()):
        r = by_case.get(case)
        if r is None or t["metric"] not in r:
            missing.append(case)
            continue
        v = float(r[t["metric"]])
        rows.append({"case": case, "metric": t["metric"], "value": v, "floor": float(t["floor"]), "ok": v >= float(t["floor"])})
    return rows, missing


def updated(results: List[dict], thresholds: Dict[str, dict], margin: float = 0.85) -> Dict[str, dict]:
    by_case = {r["case"]: r for r in results if not r.get("small")}
    out = {}
    for case, t in thresholds.items():
        r = by_case.get(case)
        out[case] = {"metric": t["metric"], "floor": round(float(r[t["metric"]]) * margin, 3)} if r and t["metric"] in r else dict(t)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("results", help="JSON written by benchmarks.kernels --out")
    ap.add_argument("--thresholds", default=DEFAULT)
    ap.add_argument("--update", action="store_true", help="rewrite the floors from these results")
    ap.add_argument("--margin", type=float, default=0.85)
    ap.add_argument("--strict", action="store_true", help="a thresholded case without a result also fails")
    a = ap.parse_args(argv)
    with open(a.results) as f:
        results = json.load(f)
    thresholds = load_thresholds(a.thresholds)
    if a.update:
        with open(a.thresholds) as f:
            about = json.load(f).get("_about", "")
        with open(a.thresholds, "w") as f:
            json.dump({"_about": about, **updated(results, thresholds, a.margin)}, f, indent=1)
        print(f"floors rewritten at {a.margin:.2f} of the measured values")
        return 0
    rows, missing = compare(results, thresholds)
    for r in rows:
        print(f"{'ok  ' if r['ok'] else 'FAIL'} {r['case']:14s} {r['metric']:26s} {r['value']:.3f} (floor {r['floor']:.3f})")
    for m in missing:
        print(f"none {m:14s} no full-size result in {a.results}")
    bad = [r for r in rows if not r["ok"]]
    return 1 if bad or (a.strict and missing) else 0


if __name__ == "__main__":
    sys.exit(main())

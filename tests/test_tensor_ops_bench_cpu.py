"""Tensor micro-benchmark list and the regression checker with the reference's thresholds."""
import copy

from sneppx_alg_b200.benchmarks import tensor_ops


def test_benchmark_rows_and_regression_thresholds():
    res = tensor_ops.run("cpu", scale_runs=0.02)
    names = [r["op"] for r in res["results"]]
    assert names == [p[0] for p in tensor_ops.PUBLISHED] and all(r["min_ms"] <= r["mean_ms"] <= r["max_ms"] for r in res["results"])
    assert all(r["vs_published"] > 0 for r in res["results"] if r["published_ms"])
    ok, rows = tensor_ops.compare(res, res)
    assert ok and all(abs(r["change"]) < 1e-12 for r in rows)
    worse = copy.deepcopy(res)
    for r in worse["results"]:
        r["min_ms"] *= 1.12  # over the 10 % GEMM / algorithm and 5 % allocator limits, under the 15 % autodiff limit
    ok, rows = tensor_ops.compare(res, worse)
    flagged = {r["category"] for r in rows if r["regressed"]}
    assert not ok and flagged == {"gemm", "allocator", "algorithms"}


def test_tiny_hybrid_parity_config_trains():
    from sneppx_alg_b200.benchmarks import tiny_hybrid
    r = tiny_hybrid.run("cpu", steps=2, warmup=1, batch=1, seq=128)
    assert r["params"] == 22512480 and 10.0 < r["ce_loss"][0] < 10.8   # ln(32000) = 10.37 at initialisation
    assert r["ce_loss"][-1] < r["ce_loss"][0] - 0.5


def test_bench_markers_on_stderr(monkeypatch, capsys):
    import torch
    from sneppx_alg_b200.algorithms.hss import HSSModel
    from sneppx_alg_b200.algorithms.ser import SERModel
    from sneppx_alg_b200.utils.observability import parse_bench_markers
    hss = HSSModel(input_dim=8, output_dim=8, state_dim=4, num_layers=1, seq_len=6)
    ser = SERModel(input_dim=8, hidden_dim=16, output_dim=8, num_experts=4, top_k=2, num_layers=2)
    x = torch.randn(2, 6, 8)
    hss(x); ser(x)
    assert "[BENCH]" not in capsys.readouterr().err                      # silent unless asked
    monkeypatch.setenv("SNEPPX_BENCH", "1")
    hss(x); ser(x)
    err = capsys.readouterr().err
    assert "[BENCH] HSS forward start\n[BENCH] HSS forward done" in err
    assert parse_bench_markers(err) == [("HSS forward", 1), ("SER layer forward", 2)]

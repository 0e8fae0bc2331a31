"""The performance regression gate: floors, comparison, update (``benchmarks/regression.py``)."""
import json

from sneppx_alg_b200.benchmarks import regression as rg


def test_floors_compare_and_update(tmp_path, capsys):
    th = rg.load_thresholds()
    assert {"gemm", "attn_fwd", "adamw", "paged_decode"} <= set(th) and all(0 < t["floor"] < 1.05 for t in th.values())
    results = [{"case": "gemm", "frac_tensor_of_measured": 0.80, "ms": 0.8}, {"case": "adamw", "frac_hbm_of_measured": 0.5},
               {"case": "ce", "frac_hbm_of_measured": 0.2, "small": True}, {"case": "unknown", "frac_hbm_of_measured": 0.1}]
    rows, missing = rg.compare(results, th)
    got = {r["case"]: r["ok"] for r in rows}
    assert got == {"gemm": True, "adamw": False} and "ce" in missing and "paged_decode" in missing
    f = tmp_path / "r.json"
    f.write_text(json.dumps(results))
    assert rg.main([str(f)]) == 1
    out = capsys.readouterr().out
    assert "FAIL adamw" in out and "ok   gemm" in out
    good = [{"case": c, t["metric"]: t["floor"] + 0.01} for c, t in th.items()]
    f.write_text(json.dumps(good))
    assert rg.main([str(f), "--strict"]) == 0
    f.write_text(json.dumps(good[:3]))
    assert rg.main([str(f)]) == 0 and rg.main([str(f), "--strict"]) == 1
    mine = tmp_path / "t.json"
    mine.write_text(json.dumps({"_about": "x", "gemm": {"metric": "frac_tensor_of_measured", "floor": 0.1},
                                "rope": {"metric": "frac_hbm_of_measured", "floor": 0.3}}))
    f.write_text(json.dumps([{"case": "gemm", "frac_tensor_of_measured": 0.9}]))
    assert rg.main([str(f), "--thresholds", str(mine), "--update", "--margin", "0.9"]) == 0
    new = json.loads(mine.read_text())
    assert new["gemm"]["floor"] == 0.81 and new["rope"]["floor"] == 0.3 and new["_about"] == "x"

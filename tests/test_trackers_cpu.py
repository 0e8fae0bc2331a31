"""Experiment trackers: the MLflow file-store layout and the W&B offline-run layout are written as those tools read them."""
import json
import os

import pytest

from sneppx_alg_b200.utils.observability import CompositeTracker, MLflowTracker, WandbTracker, make_tracker


def test_mlflow_file_store_layout(tmp_path):
    t = make_tracker("mlflow", directory=str(tmp_path), experiment="exp-a")
    assert isinstance(t, MLflowTracker)
    rid = t.start_run("run1", {"lr": 3e-4, "model/name": "tiny", "../evil": 1})
    for step in range(3):
        t.log_metrics({"loss": 2.0 - 0.5 * step, "eval/acc": 0.1 * step}, step=step)
    art = tmp_path / "note.txt"
    art.write_text("hello")
    t.log_artifact(str(art))
    t.end_run()
    root = tmp_path / "mlruns"
    exp_dirs = [d for d in os.listdir(root)]
    assert exp_dirs == ["0"]
    meta = (root / "0" / "meta.yaml").read_text()
    assert "name: exp-a\n" in meta and "experiment_id: '0'" in meta and "lifecycle_stage: active" in meta
    run = root / "0" / t.mlflow_run_id
    rmeta = (run / "meta.yaml").read_text()
    assert f"run_id: {t.mlflow_run_id}" in rmeta and "status: 3" in rmeta and "end_time: null" not in rmeta
    assert (run / "params" / "lr").read_text() == "0.0003" and (run / "params" / "model" / "name").read_text() == "tiny"
    assert not (tmp_path / "evil").exists() and (run / "params" / "_" / "evil").exists()     # keys cannot leave the run directory
    lines = (run / "metrics" / "loss").read_text().splitlines()
    assert len(lines) == 3 and [float(l.split()[1]) for l in lines] == [2.0, 1.5, 1.0] and [int(l.split()[2]) for l in lines] == [0, 1, 2]
    assert t.read_metric("eval/acc")[2][1:] == (0.2, 2)
    assert (run / "tags" / "mlflow.runName").read_text() == rid and (run / "artifacts" / "note.txt").read_text() == "hello"
    # a second run of the same experiment reuses the experiment directory; another experiment gets id 1
    t.start_run("run2")
    t.end_run("FAILED")
    assert "status: 4" in (root / "0" / t.mlflow_run_id / "meta.yaml").read_text()
    u = MLflowTracker(directory=str(tmp_path), experiment="exp-b")
    u.start_run("r")
    u.end_run()
    assert sorted(os.listdir(root)) == ["0", "1"]


def test_wandb_offline_layout_and_composite(tmp_path):
    w = WandbTracker(directory=str(tmp_path / "w"), experiment="p")
    c = CompositeTracker([w, MLflowTracker(directory=str(tmp_path / "m"), experiment="p")])
    c.start_run("r", {"bs": 8})
    c.log_metrics({"loss": 1.25}, step=5)
    c.log_metrics({"loss": 1.0, "lr": 0.1}, step=6)
    c.end_run()
    files = w.wandb_dir
    hist = [json.loads(l) for l in open(os.path.join(files, "wandb-history.jsonl"))]
    assert [h["_step"] for h in hist] == [5, 6] and hist[1]["loss"] == 1.0 and hist[1]["_runtime"] >= hist[0]["_runtime"]
    summ = json.load(open(os.path.join(files, "wandb-summary.json")))
    assert summ["loss"] == 1.0 and summ["lr"] == 0.1 and summ["_step"] == 6
    cfg = open(os.path.join(files, "config.yaml")).read()
    assert "wandb_version: 1" in cfg and "bs:\n  desc: null\n  value: 8" in cfg
    assert os.path.basename(os.path.dirname(files)).startswith("offline-run-")
    assert os.path.exists(os.path.join(str(tmp_path / "m"), "mlruns", "0"))


def test_tensorboard_event_files(tmp_path):
    """Event files written by hand: framing and checksums re-read here, content re-read by TensorBoard's own loader
    where that package is importable."""
    import glob
    import struct

    import numpy as np

    from sneppx_alg_b200.utils.observability import TensorBoardTracker, make_tracker
    assert TensorBoardTracker._crc32c(b"123456789") == 0xE3069283            # the CRC-32C check value
    t = make_tracker("tensorboard", directory=str(tmp_path))
    assert isinstance(t, TensorBoardTracker)
    t.start_run("r1", {"lr": 3e-4, "model": "tiny"})
    for i in range(5):
        t.log_metrics({"loss": 1.0 / (i + 1), "lr": 1e-3}, step=i)
    t.log_histogram("weights", np.linspace(-1, 1, 1000), step=4)
    t.end_run()
    files = glob.glob(str(tmp_path / "default" / "r1" / "events.out.tfevents.*"))
    assert len(files) == 1 and (tmp_path / "default" / "r1" / "metrics.jsonl").exists()
    raw, pos, records = open(files[0], "rb").read(), 0, []
    while pos < len(raw):
        (n,) = struct.unpack("<Q", raw[pos:pos + 8])
        assert struct.unpack("<I", raw[pos + 8:pos + 12])[0] == TensorBoardTracker._masked_crc(raw[pos:pos + 8])
        body = raw[pos + 12:pos + 12 + n]
        assert struct.unpack("<I", raw[pos + 12 + n:pos + 16 + n])[0] == TensorBoardTracker._masked_crc(body)
        records.append(body)
        pos += 16 + n
    assert len(records) == 8 and b"brain.Event:2" in records[0] and b"| lr | 0.0003 |" in records[1]
    ea = pytest.importorskip("tensorboard.backend.event_processing.event_accumulator")
    acc = ea.EventAccumulator(str(tmp_path / "default" / "r1"))
    acc.Reload()
    tags = acc.Tags()
    assert tags["scalars"] == ["loss", "lr"] and tags["histograms"] == ["weights"] and tags["tensors"] == ["parameters/text_summary"]
    assert [(s.step, round(s.value, 4)) for s in acc.Scalars("loss")] == [(0, 1.0), (1, 0.5), (2, 0.3333), (3, 0.25), (4, 0.2)]
    h = acc.Histograms("weights")[0].histogram_value
    assert h.num == 1000 and abs(h.min + 1) < 1e-9 and abs(h.max - 1) < 1e-9 and sum(h.bucket) == 1000

"""Experiment trackers: the MLflow file-store layout and the W&B offline-run layout are written as those tools read them."""
import json
import os

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

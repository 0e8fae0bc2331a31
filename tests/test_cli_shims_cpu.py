"""CLIs end to end on tiny presets, alias packages, and the added optimizers."""
import json
import os

import pytest
import torch

from sneppx_alg_b200 import cli


def test_optimizers_descend():
    from sneppx_alg_b200.optim.zoo import get_optimizer
    torch.manual_seed(0)
    for name, lr in (("sm3", 0.1), ("demeter", 0.05), ("caprop", 0.05), ("soap", 0.05), ("orthoadam", 0.05),
                     ("distributed_adam", 0.05)):
        w = torch.nn.Parameter(torch.randn(8, 6))
        b = torch.nn.Parameter(torch.zeros(6))
        x, y = torch.randn(32, 8), torch.randn(32, 6)
        opt = get_optimizer(name, [w, b], lr=lr)
        first = None
        for _ in range(40):
            loss = ((x @ w + b - y) ** 2).mean()
            opt.zero_grad()
            loss.backward()
            opt.step()
            first = first if first is not None else loss.item()
        # OrthoAdam discards the component along recent gradients, so it only has to make progress
        assert loss.item() < (0.99 if name == "orthoadam" else 0.8) * first, name


def test_alias_packages():
    import sneppx
    import SneppX_ALG
    from SneppX_ALG import interface_bindings as ib
    assert sneppx.nn.Linear is SneppX_ALG.Linear
    assert sneppx.hub is not None and sneppx.serving is not None and sneppx.distributed.get_world_size() == 1
    missing = []
    for n in ib.__all__:
        try:
            getattr(ib, n)
        except Exception as e:  # noqa: BLE001
            missing.append((n, repr(e)))
    assert not missing, missing


def test_train_eval_quantize_rlhf_experiment_cli(tmp_path, capsys):
    cfg = {"model": {"name": "llama3-tiny"}, "data": {"seq_len": 32, "length": 64},
           "training": {"batch_size": 2, "max_steps": 3, "seed": 1}, "optimizer": {"lr": 1e-3},
           "logging": {"dir": str(tmp_path / "runs"), "log_every": 1}, "checkpoint": {"dir": str(tmp_path / "ck"), "save_every": 0}}
    p = tmp_path / "cfg.json"
    p.write_text(json.dumps(cfg))
    assert cli.main(["train", "-c", str(p)]) == 0
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["steps"] == 3
    assert cli.main(["eval", "--model", "llama3-tiny", "--tasks", "mmlu", "--limit", "3"]) == 0
    res = json.loads(capsys.readouterr().out)
    assert res["mmlu"]["samples"] == 3 and res["mmlu"]["nll"] > 0
    out = tmp_path / "q.sneppx"
    assert cli.main(["quantize", "--mode", "int4", "--model-config", "llama3-tiny", "--output", str(out)]) == 0
    r = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert r["ratio"] > 1.5 and out.exists()
    assert cli.main(["rlhf", "--method", "dpo", "--model", "llama3-tiny", "--steps-per-epoch", "2"]) == 0
    assert len(json.loads(capsys.readouterr().out.strip().splitlines()[-1])["losses"]) == 2
    assert cli.main(["experiment", "--dir", str(tmp_path / "runs"), "list"]) == 0
    listing = capsys.readouterr().out
    if listing.strip():
        rid = listing.split()[0]
        assert cli.main(["experiment", "--dir", str(tmp_path / "runs"), "view", rid]) == 0
        assert cli.main(["experiment", "--dir", str(tmp_path / "runs"), "export", "--output", str(tmp_path / "e.json")]) == 0
    assert cli.main(["bogus"]) == 2


def test_serve_cli_dry_run_and_hub_cli(tmp_path, capsys):
    pytest.importorskip("fastapi")
    assert cli.main(["serve", "--model-config", "llama3-tiny", "--dry-run"]) == 0
    routes = json.loads(capsys.readouterr().out.strip().splitlines()[-1])["routes"]
    assert "/v1/generate" in routes and "/v1/chat/completions" in routes and "/v1/health" in routes
    assert cli.main(["hub", "--root", str(tmp_path / "hub"), "list"]) == 0


def test_tools_cli(tmp_path, capsys):
    import json

    import numpy as np
    import torch
    from sneppx_alg_b200.cli import tools_main
    from sneppx_alg_b200.hub import formats
    assert tools_main(["config", str(tmp_path / "train.json"), "--model", "llama3-8b"]) == 0
    cfg = json.load(open(tmp_path / "train.json"))
    assert cfg["model"]["hidden_size"] == 4096 and "optimizer" in cfg
    np.save(tmp_path / "ids.npy", np.array([1, 1, 2, 3, 3, 3], dtype=np.int32))
    capsys.readouterr()
    assert tools_main(["data", str(tmp_path / "ids.npy"), "--top", "1"]) == 0
    assert json.loads(capsys.readouterr().out)["top"] == [[3, 3]]
    (tmp_path / "t.txt").write_text("a b a\nc")
    assert tools_main(["data", str(tmp_path / "t.txt")]) == 0
    assert json.loads(capsys.readouterr().out)["distinct_words"] == 3
    sd = {"w": torch.randn(3, 4), "b": torch.zeros(4)}
    formats.save_safetensors(str(tmp_path / "m.safetensors"), sd)
    for ext in ("sneppx", "pth", "npz", "gguf", "sxh5"):
        assert tools_main(["convert", str(tmp_path / "m.safetensors"), str(tmp_path / f"m.{ext}")]) == 0
        assert torch.equal(formats.load_any(str(tmp_path / f"m.{ext}"))["w"], sd["w"])
    assert tools_main(["convert", str(tmp_path / "m.safetensors"), str(tmp_path / "m.xyz")]) == 2
    (tmp_path / "serve.json").write_text(json.dumps({"api_keys_required": True, "max_prompt_chars": 1000, "audit_log": "a.log"}))
    assert tools_main(["audit", str(tmp_path / "serve.json")]) == 0
    (tmp_path / "bad.json").write_text(json.dumps({"bind": "0.0.0.0"}))
    assert tools_main(["audit", str(tmp_path / "bad.json")]) == 1


def test_tools_card_keygen_sign_verify(tmp_path, capsys):
    import stat
    from sneppx_alg_b200.cli import tools_main
    from sneppx_alg_b200.hub.model_card import ModelCard
    assert tools_main(["card", "llama3-tiny", str(tmp_path / "card.json"), "--license", "apache-2.0"]) == 0
    card = ModelCard.load(str(tmp_path / "card.json"))
    assert card.name == "llama3-tiny" and card.num_parameters > 0 and card.license == "apache-2.0"
    assert tools_main(["card", "llama3-tiny", str(tmp_path / "card.md")]) == 0
    assert open(tmp_path / "card.md").read().startswith("# llama3-tiny 1.0.0")
    pkg = tmp_path / "update.bin"
    pkg.write_bytes(os.urandom(2048))
    for scheme in ("ml-dsa-65", "ed25519", "slh-dsa-128f"):
        prefix = str(tmp_path / scheme)
        assert tools_main(["keygen", prefix, "--scheme", scheme]) == 0
        assert stat.S_IMODE(os.stat(prefix + ".key").st_mode) == 0o600
        assert tools_main(["sign", str(pkg), prefix + ".key", "--scheme", scheme, "--version", "2.1.0"]) == 0
        manifest = str(pkg) + ".manifest.json"
        assert json.load(open(manifest))["scheme"] == scheme
        assert tools_main(["verify", str(pkg), manifest, prefix + ".pub"]) == 0
        other = str(tmp_path / (scheme + "-other"))
        tools_main(["keygen", other, "--scheme", scheme])
        assert tools_main(["verify", str(pkg), manifest, other + ".pub"]) == 1
    pkg.write_bytes(b"changed")
    assert tools_main(["verify", str(pkg), str(pkg) + ".manifest.json", str(tmp_path / "ed25519.pub")]) == 1


def test_tools_cert_issues_chains_that_tls_and_openssl_accept(tmp_path, capsys):
    import shutil
    import subprocess
    from sneppx_alg_b200.cli import tools_main
    from sneppx_alg_b200.security import tls13
    root, node = str(tmp_path / "root"), str(tmp_path / "node")
    for prefix in (root, node):
        assert tools_main(["keygen", prefix, "--scheme", "ed25519"]) == 0
    assert tools_main(["cert", root + ".key", "cluster root", root + ".pem", "--ca"]) == 0
    assert tools_main(["cert", node + ".key", "node0", node + ".der", "--dns", "node0.svc", "--dns", "*.pods.svc",
                       "--issuer-key", root + ".key", "--issuer-name", "cluster root", "--days", "30"]) == 0
    assert tools_main(["cert", node + ".key", "node0", node + ".pem", "--dns", "node0.svc",
                       "--issuer-key", root + ".key", "--issuer-name", "cluster root"]) == 0
    out = [json.loads(line) for line in capsys.readouterr().out.splitlines() if line.startswith('{"subject"')]
    assert out[0]["ca"] and out[1]["issuer"] == "cluster root" and out[1]["dns_names"] == ["node0.svc", "*.pods.svc"]
    pem = open(root + ".pem").read()
    assert pem.startswith("-----BEGIN CERTIFICATE-----\n") and all(len(l) <= 64 for l in pem.splitlines()[1:-1])
    import base64
    root_der = base64.b64decode("".join(pem.splitlines()[1:-1]))
    leaf_der = open(node + ".der", "rb").read()
    assert tls13.verify_chain([leaf_der], [root_der], "a.pods.svc") == open(node + ".pub", "rb").read()
    if shutil.which("openssl"):
        r = subprocess.run(["openssl", "verify", "-CAfile", root + ".pem", "-verify_hostname", "node0.svc", node + ".pem"],
                           capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
    with pytest.raises(SystemExit):
        tools_main(["cert", node + ".key", "x", str(tmp_path / "x.der"), "--issuer-key", root + ".key"])

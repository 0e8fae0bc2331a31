"""Command-line entry points: ``sneppx-train``, ``sneppx-serve``, ``sneppx-eval``, ``sneppx-quantize``,
``sneppx-rlhf``, ``sneppx-experiment``, ``sneppx-onnx``, ``sneppx-hub`` (the reference's ``train_cli.py``,
``serve_cli.py``, ``eval_cli.py``, ``quantize_cli.py``, ``rlhf_cli.py``, ``experiment_cli.py``, ``onnx/cli.py``,
``model_hub/cli/main.py``).  Each ``*_main(argv)`` returns a process exit code; ``main`` dispatches
``python -m sneppx_alg_b200.cli <command> ...``."""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch


def _device_dtype():
    return ("cuda", torch.bfloat16) if torch.cuda.is_available() else ("cpu", torch.float32)


def _model_from_spec(spec, dtype=None, device=None):
    """spec: preset name ('llama3-8b'), a JSON / YAML config path, or a saved-model directory."""
    from .hub.model_hub import ModelHub
    from .models import ModelConfig, build_model, create_model
    if os.path.isdir(spec):
        return ModelHub.from_pretrained(spec, dtype=dtype, device=device)
    if os.path.isfile(spec):
        import yaml
        d = yaml.safe_load(open(spec)) if spec.endswith((".yaml", ".yml")) else json.load(open(spec))
        return build_model(ModelConfig.from_dict(d), dtype=dtype, device=device)
    return create_model(spec, dtype=dtype, device=device)


# ----------------------------------------------------------------------------- train
def train_main(argv=None):
    from .training.config import TrainConfig
    from .training.data import DataLoader, MemoryMappedTextDataset, SyntheticTokenDataset
    from .training.trainer import Trainer
    ap = argparse.ArgumentParser(prog="sneppx-train", description="Train a model from a YAML / JSON config")
    ap.add_argument("--config", "-c", required=True)
    ap.add_argument("--eval-only", action="store_true")
    ap.add_argument("--resume", default=None)
    ap.add_argument("--override", "-o", default=None, help="JSON string of config overrides")
    ap.add_argument("--checkpoint-dir", default=None)
    ap.add_argument("--max-steps", type=int, default=None)
    a = ap.parse_args(argv)
    cfg = TrainConfig.load(a.config)
    if a.override:
        cfg = cfg.override(json.loads(a.override))
    if a.checkpoint_dir:
        cfg = cfg.override({"checkpoint": {"dir": a.checkpoint_dir}})
    if a.max_steps is not None:
        cfg = cfg.override({"training": {"max_steps": a.max_steps}})
    if a.resume:
        cfg = cfg.override({"checkpoint": {"resume_from": a.resume}})
    if "RANK" in os.environ and int(os.environ.get("WORLD_SIZE", "1")) > 1:
        from .parallel import distributed as sdist
        sdist.init_process_group()
    device, dtype = _device_dtype()
    m = cfg.to_dict().get("model", {})
    model = _model_from_spec(m.get("name") or m.get("config") or "llama3-tiny", dtype=dtype, device=device)
    d = cfg.to_dict().get("data", {})
    seq, bs = int(d.get("seq_len", 128)), int(cfg.training.batch_size)
    vocab = model.config.vocab_size
    if d.get("path"):
        ds = MemoryMappedTextDataset(d["path"], seq)
    else:
        ds = SyntheticTokenDataset(vocab, seq, length=int(d.get("length", 1 << 16)), seed=cfg.training.seed)
    loader = DataLoader(ds, batch_size=bs, shuffle=not a.eval_only, pin_memory=device == "cuda", seed=cfg.training.seed)
    tr = Trainer(model, cfg)
    if a.eval_only:
        print(json.dumps(tr.evaluate(loader, max_batches=int(d.get("eval_batches", 8)))))
        return 0
    out = tr.fit(loader, max_steps=cfg.training.max_steps)
    print(json.dumps({"steps": tr.step_count, **({k: v for k, v in out.items() if isinstance(v, (int, float))} if isinstance(out, dict) else {})}))
    return 0


# ----------------------------------------------------------------------------- serve
def serve_main(argv=None):
    ap = argparse.ArgumentParser(prog="sneppx-serve", description="OpenAI-shape inference server")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--log-level", default="info")
    ap.add_argument("--model-config", default="llama3-tiny", help="preset name, config file or saved-model directory")
    ap.add_argument("--model-id", default="default")
    ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--tokenizer", default=None, help="path of a BPE tokenizer file")
    ap.add_argument("--workers", type=int, default=1)
    ap.add_argument("--auth-mode", choices=["none", "api_key"], default="none")
    ap.add_argument("--api-keys", default=None, help="comma-separated keys")
    ap.add_argument("--admin-key", default=None)
    ap.add_argument("--rate-limit-rpm", type=int, default=0)
    ap.add_argument("--no-prompt-filter", action="store_true")
    ap.add_argument("--no-output-verifier", action="store_true")
    ap.add_argument("--quantize", choices=["none", "fp8", "int4"], default="none")
    ap.add_argument("--max-batch-size", type=int, default=32)
    ap.add_argument("--tls-certfile", default=None)
    ap.add_argument("--tls-keyfile", default=None)
    ap.add_argument("--dry-run", action="store_true", help="build the app and exit (used by tests)")
    ap.add_argument("--front-end", choices=["fastapi", "native"], default="fastapi",
                    help="native: the C++ HTTP server with the /v1/health, /v1/models, /v1/generate surface")
    a = ap.parse_args(argv)
    from .serving.server import create_app
    device, dtype = _device_dtype()
    model = _model_from_spec(a.model_config, dtype=dtype, device=device).eval()
    if a.checkpoint:
        from .checkpoint.sneppx_format import load_tensors
        model.load_state_dict(load_tensors(a.checkpoint)[0], strict=False)
    if a.quantize != "none":
        from .ops.quant import quantize_model_
        quantize_model_(model, a.quantize)
    spec = {"model": model, "engine_kwargs": {"max_batch_size": a.max_batch_size, "num_blocks": 256}}
    if a.tokenizer:
        from .utils.host import BPETokenizer
        tok = BPETokenizer()
        tok.load(a.tokenizer)
        spec["tokenizer"] = tok
    keys = set(a.api_keys.split(",")) if (a.auth_mode == "api_key" and a.api_keys) else None
    if a.front_end == "native":
        import time
        from .serving.native_http import TextEngine, serve_engine
        eng = TextEngine(model, spec.get("tokenizer"), a.model_id, **spec["engine_kwargs"])
        srv = serve_engine(eng, {a.model_id: {"config": a.model_config}}, token=(sorted(keys)[0] if keys else ""),
                           port=0 if a.dry_run else a.port, workers=max(a.workers, 2), host=a.host)
        print(json.dumps({"front_end": "native", "port": srv.port}), flush=True)
        try:
            while not a.dry_run:
                time.sleep(1.0)
        except KeyboardInterrupt:
            pass
        srv.stop()
        eng.stop()
        return 0
    app = create_app({a.model_id: spec}, a.model_id, api_keys=keys, admin_key=a.admin_key)
    if a.dry_run:
        print(json.dumps({"routes": sorted({r.path for r in app.routes})}))
        for w in app.state.workers.values():
            w.stop()
        return 0
    import uvicorn
    uvicorn.run(app, host=a.host, port=a.port, log_level=a.log_level, workers=1, ssl_certfile=a.tls_certfile,
                ssl_keyfile=a.tls_keyfile)
    return 0


# ----------------------------------------------------------------------------- eval
def _synthetic_task(name, vocab, n, seq, seed):
    """Stand-in task data: (prompt ids, gold next-token) pairs drawn with a task-specific seed.  Real benchmark files
    are read from ``$SNEPPX_EVAL_DATA/<task>.jsonl`` when present (lines of {"input_ids": [...], "target": id})."""
    root = os.environ.get("SNEPPX_EVAL_DATA")
    if root and os.path.exists(os.path.join(root, f"{name}.jsonl")):
        rows = [json.loads(line) for line in open(os.path.join(root, f"{name}.jsonl"))][:n]
        return [(torch.tensor(r["input_ids"]), int(r["target"])) for r in rows], "file"
    g = torch.Generator().manual_seed(seed + sum(map(ord, name)))
    return [(torch.randint(0, vocab, (seq,), generator=g), int(torch.randint(0, vocab, (1,), generator=g))) for _ in range(n)], "synthetic"


def eval_main(argv=None):
    ap = argparse.ArgumentParser(prog="sneppx-eval", description="Evaluate a model on next-token tasks")
    ap.add_argument("--model", default="llama3-tiny")
    ap.add_argument("--tasks", nargs="+", default=["mmlu", "gsm8k", "humaneval"])
    ap.add_argument("--num-fewshot", type=int, default=0)
    ap.add_argument("--limit", type=int, default=16)
    ap.add_argument("--output", default=None)
    ap.add_argument("--seed", type=int, default=42)
    a = ap.parse_args(argv)
    device, dtype = _device_dtype()
    model = _model_from_spec(a.model, dtype=dtype, device=device).eval()
    res = {}
    for task in a.tasks:
        data, src = _synthetic_task(task, model.config.vocab_size, a.limit or 16, 32 * (1 + a.num_fewshot), a.seed)
        hit, nll, t0 = 0, 0.0, time.time()
        with torch.no_grad():
            for ids, gold in data:
                logits = model(ids[None].to(device))["logits"][0, -1].float()
                hit += int(logits.argmax()) == gold
                nll += float(torch.logsumexp(logits, -1) - logits[gold])
        res[task] = {"accuracy": hit / len(data), "nll": nll / len(data), "samples": len(data), "data": src,
                     "seconds": time.time() - t0}
    txt = json.dumps(res, indent=1)
    if a.output:
        open(a.output, "w").write(txt)
    print(txt)
    return 0


# ----------------------------------------------------------------------------- quantize
def quantize_main(argv=None):
    ap = argparse.ArgumentParser(prog="sneppx-quantize", description="Quantise a model's linear layers")
    ap.add_argument("--mode", default="int4", choices=["int4", "int8", "fp8", "awq", "gptq"])
    ap.add_argument("--granularity", default="per_channel", choices=["per_tensor", "per_channel"])
    ap.add_argument("--model-config", required=True)
    ap.add_argument("--output", default=None)
    ap.add_argument("--skip-layers", nargs="*", default=["lm_head", "embed_tokens", "embedding"])
    a = ap.parse_args(argv)
    from . import quant as Q
    from .checkpoint.sneppx_format import save_tensors
    device, dtype = _device_dtype()
    model = _model_from_spec(a.model_config, dtype=dtype, device=device)
    out, before, after = {}, 0, 0
    for name, p in model.state_dict().items():
        w = p.detach()
        before += w.numel() * w.element_size()
        skip = w.dim() != 2 or any(s in name for s in a.skip_layers) or w.shape[-1] % 128
        if skip:
            out[name] = w.cpu()
        elif a.mode == "int8":
            mode = Q.QuantMode.INT8_PER_CHANNEL if a.granularity == "per_channel" else Q.QuantMode.INT8_SYMMETRIC
            q, s, _ = Q.quantize_int8(w, mode)
            out[name + ".q"], out[name + ".scale"] = q.cpu(), s.float().reshape(-1).cpu()
        elif a.mode == "fp8":
            q, s = Q.quant_fp8_128x128(w.to(torch.bfloat16)) if w.is_cuda else Q.quantize_fp8(w)
            out[name + ".q"], out[name + ".scale"] = q.view(torch.uint8).cpu(), torch.as_tensor(s).float().reshape(-1).cpu()
        else:
            if a.mode == "awq":
                w = Q.awq_quantize(w.float(), w.float().abs().mean(0))[0]
            elif a.mode == "gptq":
                w = Q.gptq_quantize(w.float(), torch.randn(256, w.shape[1], device=w.device))
            q, s = Q.quantize_int4_packed(w.float())
            out[name + ".q"], out[name + ".scale"] = q.cpu(), s.float().cpu()
        if not skip:
            after += sum(out[name + k].numel() * out[name + k].element_size() for k in (".q", ".scale"))
        else:
            after += w.numel() * w.element_size()
    if a.output:
        save_tensors(a.output, out, metadata={"quantization": a.mode, "granularity": a.granularity})
    print(json.dumps({"mode": a.mode, "bytes_before": before, "bytes_after": after, "ratio": before / max(after, 1),
                      "output": a.output}))
    return 0


# ----------------------------------------------------------------------------- rlhf
def rlhf_main(argv=None):
    ap = argparse.ArgumentParser(prog="sneppx-rlhf", description="Preference optimisation (DPO / GRPO)")
    ap.add_argument("--method", default="dpo", choices=["dpo", "grpo"])
    ap.add_argument("--model", default="llama3-tiny")
    ap.add_argument("--learning-rate", type=float, default=1e-5)
    ap.add_argument("--beta", type=float, default=0.1)
    ap.add_argument("--group-size", type=int, default=8)
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--steps-per-epoch", type=int, default=4)
    ap.add_argument("--data", default=None, help="JSONL of {chosen: [...], rejected: [...]} (DPO) or {prompt: [...]} (GRPO)")
    ap.add_argument("--output", default=None)
    a = ap.parse_args(argv)
    from .training.lora import DPOTrainer, GRPOTrainer
    device, dtype = _device_dtype()
    model = _model_from_spec(a.model, dtype=dtype, device=device)
    V = model.config.vocab_size
    rows = [json.loads(line) for line in open(a.data)] if a.data else None
    g = torch.Generator().manual_seed(0)
    hist = []
    if a.method == "dpo":
        tr = DPOTrainer(model, beta=a.beta, lr=a.learning_rate)
        for step in range(a.epochs * a.steps_per_epoch):
            if rows:
                r = rows[step % len(rows)]
                ch, rj = torch.tensor([r["chosen"]]), torch.tensor([r["rejected"]])
            else:
                ch, rj = torch.randint(0, V, (2, 16), generator=g), torch.randint(0, V, (2, 16), generator=g)
            hist.append(tr.step(ch.to(device), rj.to(device))[0])
    else:
        tr = GRPOTrainer(model, reward_fn=lambda seqs: -(seqs.float().diff(dim=-1).abs().mean(-1)) / V,
                         group_size=a.group_size, kl_coef=a.beta, lr=a.learning_rate)
        for step in range(a.epochs * a.steps_per_epoch):
            pr = torch.tensor(rows[step % len(rows)]["prompt"]) if rows else torch.randint(0, V, (8,), generator=g)
            hist.append(tr.step(pr.to(device)[None] if pr.dim() == 1 else pr.to(device))[0])
    if a.output:
        from .hub.model_hub import ModelHub
        ModelHub.save_pretrained(model, a.output)
    print(json.dumps({"method": a.method, "losses": hist}))
    return 0


# ----------------------------------------------------------------------------- experiment
def experiment_main(argv=None):
    ap = argparse.ArgumentParser(prog="sneppx-experiment", description="Inspect local experiment runs")
    ap.add_argument("--dir", default="runs")
    sub = ap.add_subparsers(dest="cmd", required=True)
    lp = sub.add_parser("list")
    lp.add_argument("--experiment", default=None)
    vp = sub.add_parser("view")
    vp.add_argument("run_id")
    cp = sub.add_parser("compare")
    cp.add_argument("run_ids", nargs="+")
    dp = sub.add_parser("delete")
    dp.add_argument("run_id")
    ep = sub.add_parser("export")
    ep.add_argument("--output", default="experiments_export.json")
    ep.add_argument("--experiment", default=None)
    a = ap.parse_args(argv)

    def runs():
        """runs/<experiment>/<run_id>/{params.json, metrics.jsonl} as the local tracker writes them."""
        out = {}
        for root, _, files in os.walk(a.dir):
            if "metrics.jsonl" in files:
                rid = os.path.basename(root)
                params = json.load(open(os.path.join(root, "params.json"))) if "params.json" in files else {}
                metrics = [json.loads(line) for line in open(os.path.join(root, "metrics.jsonl")) if line.strip()]
                out[rid] = {"run_id": rid, "experiment": os.path.basename(os.path.dirname(root)), "params": params,
                            "metrics": metrics, "status": "finished", "_path": root}
        return out

    rs = runs()
    if a.cmd == "list":
        for rid, r in sorted(rs.items()):
            if a.experiment in (None, r.get("experiment")):
                print(f"{rid}\t{r.get('experiment')}\t{r.get('status')}\t{len(r.get('metrics', []))} metric rows")
    elif a.cmd == "view":
        print(json.dumps({k: v for k, v in rs[a.run_id].items() if k != "_path"}, indent=1))
    elif a.cmd == "compare":
        keys = sorted({k for rid in a.run_ids for k in rs[rid].get("params", {})})
        for k in keys:
            print(k, *[rs[rid].get("params", {}).get(k) for rid in a.run_ids], sep="\t")
        for rid in a.run_ids:
            last = (rs[rid].get("metrics") or [{}])[-1]
            print(rid, json.dumps(last))
    elif a.cmd == "delete":
        import shutil
        shutil.rmtree(rs[a.run_id]["_path"])
    elif a.cmd == "export":
        sel = [{k: v for k, v in r.items() if k != "_path"} for r in rs.values() if a.experiment in (None, r.get("experiment"))]
        json.dump(sel, open(a.output, "w"), indent=1)
        print(f"exported {len(sel)} runs to {a.output}")
    return 0


# ----------------------------------------------------------------------------- onnx / hub
def onnx_main(argv=None):
    ap = argparse.ArgumentParser(prog="sneppx-onnx", description="ONNX toolkit: check / infer-shapes / optimize / quantize / run")
    ap.add_argument("cmd", choices=["check", "shapes", "optimize", "quantize", "info"])
    ap.add_argument("model")
    ap.add_argument("--output", default=None)
    a = ap.parse_args(argv)
    from .onnx import toolkit as T
    m = T.Model.load(a.model)
    if a.cmd == "check":
        problems = T.check_model(m)
        print(json.dumps({"ok": not problems, "problems": problems}))
        return 0 if not problems else 1
    if a.cmd == "info":
        print(json.dumps({"nodes": len(m.graph.nodes), "inputs": [i.name for i in m.graph.inputs],
                          "outputs": [o.name for o in m.graph.outputs], "initializers": len(m.graph.initializers)}))
        return 0
    if a.cmd == "shapes":
        print(json.dumps({k: list(v) for k, v in T.infer_shapes(m).items()}))
        return 0
    out = T.optimize(m) if a.cmd == "optimize" else T.quantize_qdq(m)
    out.save(a.output or a.model.replace(".onnx", f".{a.cmd}.onnx"))
    print(json.dumps({"nodes_before": len(m.graph.nodes), "nodes_after": len(out.graph.nodes)}))
    return 0


def hub_main(argv=None):
    ap = argparse.ArgumentParser(prog="sneppx-hub", description="Local model registry and registry-service client")
    ap.add_argument("--root", default="~/.sneppx/hub")
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("list")
    sp = sub.add_parser("search")
    sp.add_argument("query", nargs="?", default="")
    sp.add_argument("--tag", default=None)
    up = sub.add_parser("upload")
    up.add_argument("model_dir")
    up.add_argument("model_id")
    up.add_argument("--version", default="1.0.0")
    up.add_argument("--tags", nargs="*", default=[])
    dp = sub.add_parser("download")
    dp.add_argument("model_id")
    dp.add_argument("--version", default=None)
    lb = sub.add_parser("leaderboard")
    lb.add_argument("metric")
    cv = sub.add_parser("convert", help="convert a Hugging Face safetensors checkpoint")
    cv.add_argument("src")
    cv.add_argument("dst")
    cv.add_argument("--preset", required=True)
    # verbs against a registry service (hub/registry_server.py); the session token is kept in <root>/session.json
    sv = sub.add_parser("serve", help="run the registry service")
    sv.add_argument("--data", default="~/.sneppx/hub-server")
    sv.add_argument("--port", type=int, default=8090)
    sv.add_argument("--dry-run", action="store_true")
    for name in ("register", "login"):
        rp = sub.add_parser(name)
        rp.add_argument("url")
        rp.add_argument("username")
        rp.add_argument("password")
    sub.add_parser("logout")
    sub.add_parser("whoami")
    cr = sub.add_parser("create")
    cr.add_argument("model_id")
    cr.add_argument("--description", default="")
    cr.add_argument("--tags", nargs="*", default=[])
    cr.add_argument("--private", action="store_true")
    pu = sub.add_parser("push")
    pu.add_argument("model_dir")
    pu.add_argument("model_id")
    pu.add_argument("--version", default="1.0.0")
    pu.add_argument("--metric", action="append", default=[], help="name=value")
    pl = sub.add_parser("pull")
    pl.add_argument("model_id")
    pl.add_argument("dest")
    pl.add_argument("--version", default=None)
    inf = sub.add_parser("info")
    inf.add_argument("model_id")
    rm = sub.add_parser("delete")
    rm.add_argument("model_id")
    rs = sub.add_parser("remote-search")
    rs.add_argument("query", nargs="?", default="")
    rs.add_argument("--tag", default="")
    ky = sub.add_parser("key")
    ky.add_argument("name")
    a = ap.parse_args(argv)
    from .hub.model_hub import Hub, convert_hf_to_sneppx
    hub = Hub(a.root)
    session_path = os.path.join(hub.root, "session.json")
    if a.cmd == "serve":
        import time
        from .hub.registry_server import serve_hub
        srv = serve_hub(os.path.expanduser(a.data), 0 if a.dry_run else a.port)
        print(json.dumps({"hub": f"http://127.0.0.1:{srv.port}"}), flush=True)
        try:
            while not a.dry_run:
                time.sleep(1.0)
        except KeyboardInterrupt:
            pass
        srv.stop()
        return 0
    if a.cmd in ("register", "login", "logout", "whoami", "create", "push", "pull", "info", "delete", "remote-search", "key"):
        from .hub.registry_server import HubClient
        sess = json.load(open(session_path)) if os.path.exists(session_path) else {}
        if a.cmd in ("register", "login"):
            cl = HubClient(a.url)
            if a.cmd == "register":
                cl.register(a.username, a.password)
            json.dump({"url": a.url, "user": a.username, "token": cl.login(a.username, a.password)}, open(session_path, "w"))
            print(json.dumps({"user": a.username, "url": a.url}))
            return 0
        if a.cmd == "logout":
            if os.path.exists(session_path):
                os.remove(session_path)
            return 0
        if not sess:
            print("not logged in: run `sneppx-hub login <url> <user> <password>` first", file=sys.stderr)
            return 1
        cl = HubClient(sess["url"], sess["token"])
        if a.cmd == "whoami":
            out = {"user": sess["user"], "url": sess["url"]}
        elif a.cmd == "create":
            out = cl.create_model(a.model_id, a.description, a.tags, a.private)
        elif a.cmd == "push":
            metrics = {k: float(v) for k, v in (m.split("=", 1) for m in a.metric)}
            out = {"uploaded": cl.upload(a.model_dir, a.model_id, a.version, metrics)}
        elif a.cmd == "pull":
            out = {"path": cl.download(a.model_id, a.dest, a.version)}
        elif a.cmd == "info":
            out = cl.model_info(a.model_id)
        elif a.cmd == "delete":
            out = cl.delete_model(a.model_id)
        elif a.cmd == "remote-search":
            out = cl.search(a.query, a.tag)
        else:
            out = {"key": cl.create_api_key(a.name)}
        print(json.dumps(out, indent=1))
        return 0
    if a.cmd == "list":
        print(json.dumps(hub.list_models(), indent=1))
    elif a.cmd == "search":
        print(json.dumps(hub.search(a.query, a.tag), indent=1))
    elif a.cmd == "upload":
        print(json.dumps(hub.upload(a.model_dir, a.model_id, a.version, a.tags)))
    elif a.cmd == "download":
        print(hub.download(a.model_id, a.version))
    elif a.cmd == "leaderboard":
        print(json.dumps(hub.leaderboard(a.metric), indent=1))
    elif a.cmd == "convert":
        from .hub.formats import load_safetensors
        from .models import config_from_name
        convert_hf_to_sneppx(load_safetensors(a.src)[0], a.dst, config_from_name(a.preset))
        print(a.dst)
    return 0


# ----------------------------------------------------------------------------- tools
def tools_main(argv=None):
    """Small utilities in the place of the reference's ``tools/`` programs: config generator, data explorer, model
    converter, benchmarking suite, security auditor."""
    ap = argparse.ArgumentParser(prog="sneppx-tools", description=tools_main.__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    cg = sub.add_parser("config", help="write a training configuration template")
    cg.add_argument("out")
    cg.add_argument("--model", default="llama3-8b")
    de = sub.add_parser("data", help="statistics of a text file or a token file (.npy / .bin of int32)")
    de.add_argument("path")
    de.add_argument("--top", type=int, default=10)
    cv = sub.add_parser("convert", help="convert a weight file between .safetensors / .sneppx / .pth / .npz / .gguf / .sxh5")
    cv.add_argument("src")
    cv.add_argument("dst")
    cv.add_argument("--q8", action="store_true", help="store matrices as 8-bit blocks when the target is .gguf")
    cd = sub.add_parser("card", help="write a model card (JSON, or Markdown for a .md target) for a preset or a saved model")
    cd.add_argument("model")
    cd.add_argument("out")
    cd.add_argument("--name", default=None)
    cd.add_argument("--version", default="1.0.0")
    cd.add_argument("--license", default="")
    kg = sub.add_parser("keygen", help="signing key pair (ed25519 or post-quantum ml-dsa-65) written as <prefix>.pub / <prefix>.key")
    kg.add_argument("prefix")
    kg.add_argument("--scheme", default="ml-dsa-65", choices=["ed25519", "ml-dsa-65", "slh-dsa-128f"])
    ce = sub.add_parser("cert", help="X.509 certificate (DER, or PEM for a .pem target) for an ed25519 key made by keygen: "
                        "self-signed, or issued by --issuer-key / --issuer-name; for security.tls13 and OpenSSL alike")
    ce.add_argument("key", help="the subject's ed25519 private key file (32 bytes)")
    ce.add_argument("subject", help="common name")
    ce.add_argument("out")
    ce.add_argument("--dns", action="append", default=[], help="DNS name the certificate covers (repeatable)")
    ce.add_argument("--ca", action="store_true", help="mark as a certificate authority")
    ce.add_argument("--issuer-key", default=None)
    ce.add_argument("--issuer-name", default=None)
    ce.add_argument("--days", type=float, default=365.0)
    sg = sub.add_parser("sign", help="signed manifest for a file (update package, weight file)")
    sg.add_argument("file")
    sg.add_argument("key")
    sg.add_argument("--scheme", default="ml-dsa-65", choices=["ed25519", "ml-dsa-65", "slh-dsa-128f"])
    sg.add_argument("--version", default="1.0.0")
    sg.add_argument("--out", default=None)
    vf = sub.add_parser("verify", help="check a file against its signed manifest; exit code 0 when it is authentic")
    vf.add_argument("file")
    vf.add_argument("manifest")
    vf.add_argument("pub")
    be = sub.add_parser("bench", help="tensor micro-benchmarks (the reference's published list)")
    be.add_argument("--device", default="cpu")
    be.add_argument("--out", default=None)
    au = sub.add_parser("audit", help="security self-audit of a serving configuration file")
    au.add_argument("config")
    a = ap.parse_args(argv)
    if a.cmd == "config":
        from .models import config_from_name
        from .training.config import TrainConfig
        cfg = TrainConfig().to_dict()
        cfg["model"] = config_from_name(a.model).to_dict()
        with open(a.out, "w") as f:
            if a.out.endswith((".yaml", ".yml")):
                import yaml
                yaml.safe_dump(cfg, f, sort_keys=False)
            else:
                json.dump(cfg, f, indent=1)
        print(a.out)
    elif a.cmd == "data":
        import collections
        import numpy as np
        if a.path.endswith((".npy", ".bin")):
            ids = np.load(a.path) if a.path.endswith(".npy") else np.fromfile(a.path, dtype=np.int32)
            ids = ids.reshape(-1)
            vals, counts = np.unique(ids, return_counts=True)
            order = np.argsort(-counts)[: a.top]
            out = {"tokens": int(ids.size), "distinct": int(vals.size), "min": int(ids.min()), "max": int(ids.max()),
                   "top": [[int(vals[i]), int(counts[i])] for i in order]}
        else:
            text = open(a.path, encoding="utf-8", errors="replace").read()
            words = text.split()
            out = {"bytes": len(text.encode()), "lines": text.count("\n") + 1, "words": len(words),
                   "distinct_words": len(set(words)), "top": collections.Counter(words).most_common(a.top)}
        print(json.dumps(out, indent=1))
    elif a.cmd == "convert":
        from .checkpoint.sneppx_format import save_tensors
        from .hub import formats
        sd = formats.load_any(a.src)
        d = a.dst.lower()
        if d.endswith(".safetensors"):
            formats.save_safetensors(a.dst, {k: v.contiguous() for k, v in sd.items()})
        elif d.endswith(".sneppx"):
            save_tensors(a.dst, sd, {"source": os.path.basename(a.src)})
        elif d.endswith((".pth", ".pt")):
            formats.save_pth(a.dst, sd)
        elif d.endswith(".npz"):
            formats.save_npz(a.dst, sd)
        elif d.endswith(".gguf"):
            from .hub.model_card import save_gguf
            save_gguf(a.dst, sd, {"general.name": os.path.basename(a.src)}, q8_0=a.q8)
        elif d.endswith(".sxh5"):
            with formats.HierarchicalFile(a.dst, "w") as f:
                f.write_state_dict(sd)
        else:
            print(f"unknown target format: {a.dst}", file=sys.stderr)
            return 2
        print(json.dumps({"tensors": len(sd), "dst": a.dst}))
    elif a.cmd == "card":
        from .hub.model_card import ModelCard
        model = _model_from_spec(a.model)
        card = ModelCard.from_model(model, a.name or os.path.basename(a.model.rstrip("/")), a.version, license=a.license,
                                    model_type="causal-lm")
        ok, errors = card.validate()
        if not ok:
            print("; ".join(errors), file=sys.stderr)
            return 1
        with open(a.out, "w") as f:
            f.write(card.to_markdown() if a.out.endswith(".md") else card.to_json())
        print(a.out)
    elif a.cmd == "keygen":
        from .security import crypto
        if a.scheme == "ed25519":
            key = os.urandom(32)
            pub = crypto.ed25519_public_key(key)
        elif a.scheme == "slh-dsa-128f":
            pub, key = crypto.slhdsa_keygen("128f")
        else:
            pub, key = crypto.mldsa_keygen(65)
        with open(a.prefix + ".pub", "wb") as f:
            f.write(pub)
        fd = os.open(a.prefix + ".key", os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o600)     # private key: owner only
        with os.fdopen(fd, "wb") as f:
            f.write(key)
        print(json.dumps({"scheme": a.scheme, "public": a.prefix + ".pub", "private": a.prefix + ".key", "public_bytes": len(pub)}))
    elif a.cmd == "cert":
        import base64
        from .security import tls13
        seed = open(a.key, "rb").read()
        if len(seed) != 32:
            ap.error("certificates are issued for ed25519 keys (a 32-byte private key file)")
        if bool(a.issuer_key) != bool(a.issuer_name):
            ap.error("--issuer-key and --issuer-name go together")
        der = tls13.make_certificate(seed, a.subject, issuer_seed=open(a.issuer_key, "rb").read() if a.issuer_key else None,
                                     issuer=a.issuer_name, days=a.days, dns_names=a.dns, ca=a.ca)
        with open(a.out, "wb") as f:
            if a.out.endswith(".pem"):
                body = base64.encodebytes(der).decode().replace("\n", "")
                f.write(("-----BEGIN CERTIFICATE-----\n" + "\n".join(body[i:i + 64] for i in range(0, len(body), 64))
                         + "\n-----END CERTIFICATE-----\n").encode())
            else:
                f.write(der)
        info = tls13.parse_certificate(der)
        print(json.dumps({"subject": info["subject"], "issuer": info["issuer"], "dns_names": info["dns_names"], "ca": info["ca"],
                          "not_after": time.strftime("%Y-%m-%d", time.gmtime(info["not_after"])), "out": a.out}))
    elif a.cmd == "sign":
        from .security.services import sign_update
        manifest = sign_update(a.file, open(a.key, "rb").read(), a.version, scheme=a.scheme)
        out = a.out or a.file + ".manifest.json"
        with open(out, "w") as f:
            json.dump(manifest, f, indent=1)
        print(out)
    elif a.cmd == "verify":
        from .security.services import verify_update
        ok = verify_update(a.file, json.load(open(a.manifest)), open(a.pub, "rb").read())
        print(json.dumps({"authentic": bool(ok)}))
        return 0 if ok else 1
    elif a.cmd == "bench":
        from .benchmarks import tensor_ops
        return tensor_ops.main(["--device", a.device] + (["--out", a.out] if a.out else []))
    elif a.cmd == "audit":
        from .security.services import self_audit
        cfg = json.load(open(a.config)) if a.config.endswith(".json") else __import__("yaml").safe_load(open(a.config))
        findings = self_audit(cfg)
        print(json.dumps({"findings": findings}, indent=1))
        return 1 if findings else 0
    return 0


COMMANDS = {"train": train_main, "serve": serve_main, "eval": eval_main, "quantize": quantize_main, "rlhf": rlhf_main,
            "experiment": experiment_main, "onnx": onnx_main, "hub": hub_main, "tools": tools_main}


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] not in COMMANDS:
        print("usage: python -m sneppx_alg_b200.cli {" + ",".join(COMMANDS) + "} ...")
        return 2
    return COMMANDS[argv[0]](argv[1:])


if __name__ == "__main__":
    sys.exit(main())

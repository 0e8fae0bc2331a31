#!/usr/bin/env python
"""Headline benchmark: training tokens/s of the Llama-3-8B-shape decoder (bf16, ZeRO-3 data parallel,
seq 4096, micro-batch 1 per GPU, AdamW beta 0.9/0.95 wd 0.1), synthetic token ids, random-init weights.

    python bench.py --gpus N --steps K --warmup W          # N > 1: launched by torch.distributed.run
    python bench.py --impl reference ...                    # the unmodified reference, driven through its own API
    python bench.py --impl library ...                      # PyTorch library ops + NCCL only, overlapped like FSDP
    python bench.py --model deepseek-v2-lite --ep --micro-batch 2      # SER MoE, expert parallel + ZeRO-1
    python bench.py --model mamba2-2.7b --seq 8192 --tp 2              # Mamba-2, tensor parallel x data parallel

Rank 0 prints one JSON line. ``value`` is whole-job tokens/s from CUDA-event timing (max over ranks);
``e2e`` repeats the measurement through the public engine API with the per-step host->device copy of the
batch from pinned memory and the device->host read of the loss inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "library"])
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--layers", type=int, default=0, help="debug only: override depth (result is marked invalid)")
    ap.add_argument("--ep", action="store_true", help="expert parallelism over all ranks (SER MoE models): experts are "
                    "sharded, the other parameters use ZeRO-1")
    ap.add_argument("--zero-stage", type=int, default=3)
    ap.add_argument("--param-slots", type=int, default=0,
                    help="ZeRO-3 with sharded parameters: keep this many rotating layer slots instead of all gathered "
                         "parameters (N > 1); 0 keeps them all resident")
    ap.add_argument("--fp8-experts", action="store_true", help="SER MoE models: forward expert GEMMs in block-scaled "
                    "fp8 (e4m3 data, 1x128 activation and 128x128 weight scales); backward stays bf16")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel size (Mamba-2 models): ranks form world/tp "
                    "data-parallel replicas of tp consecutive ranks; ignored on one GPU")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], 0, set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = max(mx, float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        med = sm[len(sm) // 2] if sm else None
        return {"sm_mhz": med, "sm_max_mhz": mx or None, "reasons": sorted(reasons), "samples": len(sm)}


def run_reference(args):
    """Runs the unmodified reference (``baseline/_ref``) through its own public API in a child process
    (``baseline/reference_probe.py``) and reports what happened. The named config cannot run on it: its Llama class
    raises in forward, its generic Transformer "trains" without any parameter receiving a gradient, its tensors are
    NumPy arrays on the host whatever ``.cuda()`` says, and its collectives return their input. The line carries
    the captured observations, not a canned text."""
    ref_dir = os.path.join(REPO, "baseline", "_ref")
    probe = os.path.join(REPO, "baseline", "reference_probe.py")
    out = {"impl": "reference"}
    if not os.path.isdir(os.path.join(ref_dir, "SneppX_ALG")):
        out["unavailable"] = ("reference not installed under baseline/_ref (offline pip install of the reference source "
                              "tree not done on this box)")
        print(json.dumps(out))
        return 0
    rank = int(os.environ.get("RANK", "0"))
    obs, err = None, None
    try:
        env = {k: v for k, v in os.environ.items() if k not in ("PYTHONPATH",)}
        r = subprocess.run([sys.executable, probe], capture_output=True, text=True, timeout=600, cwd=ref_dir, env=env)
        lines = [ln for ln in r.stdout.strip().splitlines() if ln.startswith("{")]
        obs = json.loads(lines[-1]) if lines else None
        if obs is None:
            err = (r.stderr or r.stdout).strip().splitlines()[-1:] or ["no output"]
    except Exception as e:  # noqa: BLE001
        err = [f"{type(e).__name__}: {e}"]
    if obs is None:
        out["unavailable"] = f"reference probe failed: {err[0]}"
    else:
        tt = obs.get("transformer_train")
        trains = isinstance(tt, dict) and tt.get("params_changed_by_adamw_step", 0) > 0
        out["unavailable"] = (
            "the unmodified reference cannot run Llama-3-8B-shape bf16 ZeRO-3 training on GPUs: "
            f"LlamaForCausalLM forward -> {obs.get('llama_forward')}; generic Transformer step "
            f"{'updates' if trains else 'updates no'} parameters "
            f"({tt.get('params_with_grad_after_backward') if isinstance(tt, dict) else tt} of "
            f"{tt.get('params') if isinstance(tt, dict) else '?'} got a gradient); Tensor.cuda() keeps data in "
            f"{obs.get('cuda_tensor', {}).get('storage_type') if isinstance(obs.get('cuda_tensor'), dict) else obs.get('cuda_tensor')}; "
            f"all_reduce changed values: {obs.get('collectives', {}).get('all_reduce_changed_values') if isinstance(obs.get('collectives'), dict) else obs.get('collectives')}; "
            "its CUDA / NCCL C layers do not compile")
        out["observed"] = obs
    if rank == 0:
        print(json.dumps(out))
    return 0


def _dist_setup():
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    return world, rank, local_rank, dev


def measure(args, world, rank, local_rank, dev, step, vocab, B, S, data_seed, launches=None, check=None, drain=None):
    """Warm-up, the device-timed region (inputs resident on the device) and the end-to-end region (every step copies
    its batch from pinned host memory and reads the loss back), each bracketed by barrier + synchronize and timed with
    CUDA events; returns max-over-ranks milliseconds. ``step(ids) -> loss tensor``. ``drain``: makes the timing stream
    wait for work the engine still has in flight on its own streams (deferred parameter updates), called before each
    closing event so that the timed region holds all the work of its steps."""
    import torch
    import torch.distributed as dist
    gen = torch.Generator().manual_seed(data_seed)
    n_batches = args.warmup + 2 * args.steps + 2
    host = [torch.randint(0, vocab, (B, S), generator=gen, dtype=torch.int64).pin_memory() for _ in range(n_batches)]
    devb = [h.to(dev, non_blocking=True) for h in host]
    torch.cuda.synchronize()

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    it = 0
    for _ in range(args.warmup):
        step(devb[it])
        it += 1
    if check:
        check()
    torch.cuda.reset_peak_memory_stats(dev)       # peak memory of the steps, not of building the model
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    l0 = launches() if launches else 0
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step(devb[it])
        it += 1
    if drain:
        drain()
    e1.record()
    sync()
    ms = e0.elapsed_time(e1)
    n_launch = (launches() - l0) if launches else 0
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    last = 0.0
    for _ in range(args.steps):
        last = float(step(host[it].to(dev, non_blocking=True)).item())
        it += 1
    if drain:
        drain()
    f1.record()
    sync()
    ms_e2e = f0.elapsed_time(f1)
    clocks = sampler.stop() if rank == 0 else None
    if check:
        check()
    peak = torch.cuda.max_memory_allocated(dev) / 2 ** 30
    t = torch.tensor([ms, ms_e2e, peak], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e, peak = t.tolist()
    return {"ms": ms, "ms_e2e": ms_e2e, "last": last, "clocks": clocks, "launches": n_launch, "peak_gib": peak}


def model_label(cfg, args):
    name = f"{cfg.name}-shape".replace("llama3-8B", "llama3-8b")
    return name if not args.layers else f"{name}-{args.layers}L(debug, invalid)"


def result_line(args, world, dp, res, B, S, impl, model, parallelism, launches, extra_cfg=None):
    tokens = B * S * dp * args.steps
    line = {
        "metric": "train tokens/sec", "value": tokens / (res["ms"] / 1e3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms"] / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random-init weights",
        "impl": impl,
        "config": {"model": model, "global_batch": B * dp, "seq_len": S, "parallelism": parallelism,
                   "optimizer": "AdamW b=(0.9,0.95) wd=0.1 fp32 master+moments, clip 1.0",
                   "l2": "per-step working set (GBs of weights and activations) far exceeds the 126 MB L2",
                   "peak_memory_gib_per_gpu": round(res["peak_gib"], 2)},
        "e2e": {"value": tokens / (res["ms_e2e"] / 1e3), "unit": "tokens/s", "ms_per_step": res["ms_e2e"] / args.steps,
                "h2d_bytes_per_step": B * S * 8, "d2h_bytes_per_step": 4, "last_loss": res["last"]},
        "gpu_launches": launches, "clocks": res["clocks"]}
    if extra_cfg:
        line["config"].update(extra_cfg)
    return line


def run_library(args):
    """The same step stated with PyTorch library ops only (cuBLAS through F.linear / einsum, SDPA attention, F.rms_norm,
    F.conv1d, F.cross_entropy, NCCL reduce-scatter / all-gather / all-to-all, torch's fused AdamW on fp32 master
    shards), with the communication overlapped the way stock FSDP does it: the comparator this repository can actually
    run on the box, since the reference cannot run the config. Same model shapes, dtype recipe, clipping and timing
    rules as the main arm; none of this repository's kernels are on the path (``benchmarks/library_arm.py``)."""
    import torch
    import torch.distributed as dist
    world, rank, local_rank, dev = _dist_setup()
    from sneppx_alg_b200.benchmarks import library_arm
    from sneppx_alg_b200.models import config_from_name
    cfg = config_from_name(args.model)
    torch.manual_seed(1234)
    tp = args.tp if world > 1 else 1
    model, engine, par, dp, tp_group = library_arm.build(args.model, cfg, dev, world, rank, layers=args.layers, tp=tp,
                                                         ep=args.ep)
    B, S = args.micro_batch, args.seq
    dp_rank = rank // tp if tp_group is not None else rank
    def step(ids):
        loss = engine.step(ids)
        if tp_group is not None:      # each tensor-parallel rank holds its token rows' share of the mean loss
            loss = loss.clone()
            dist.all_reduce(loss, group=tp_group)
        return loss

    res = measure(args, world, rank, local_rank, dev, step, cfg.vocab_size, B, S, 100 + dp_rank)
    if rank == 0:
        print(json.dumps(result_line(
            args, world, dp, res, B, S,
            "library (PyTorch ops: cuBLAS, SDPA, NCCL, torch fused AdamW; none of this repository's kernels)",
            model_label(cfg, args), par, 0)))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main():
    args = parse()
    if args.impl == "reference":
        return run_reference(args)
    if args.impl == "library":
        return run_library(args)

    import torch
    import torch.distributed as dist
    world, rank, local_rank, dev = _dist_setup()

    from sneppx_alg_b200.models import config_from_name, build_model
    from sneppx_alg_b200.ops import _lib, check_status
    from sneppx_alg_b200.parallel.zero import make_engine

    cfg = config_from_name(args.model)
    if args.layers:
        cfg.num_hidden_layers = cfg.num_layers = args.layers
    cfg.max_position_embeddings = max(args.seq, 8)
    if args.fp8_experts:
        cfg.expert_fp8 = True
    torch.manual_seed(1234)
    arch = getattr(cfg, "architecture", "transformer")
    B, S, V = args.micro_batch, args.seq, cfg.vocab_size
    dp, dp_rank, extra = world, rank, {}
    kw = dict(lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, max_grad_norm=1.0)
    if arch == "mamba2" and world > 1 and args.tp > 1:
        # tensor parallel x data parallel: in_proj all-gather -> GEMM, out_proj GEMM -> reduce-scatter (fused kernels)
        from sneppx_alg_b200.parallel.tp import TPContext
        from sneppx_alg_b200.parallel.tp_engine import TPDPEngine, make_tp_dp_groups
        from sneppx_alg_b200.parallel.tp_mamba import TPMamba2ForCausalLM
        tp_group, dp_group, tp_rank, dp_rank = make_tp_dp_groups(args.tp)
        dp = world // args.tp
        full = build_model(cfg, dtype=torch.bfloat16, device=dev)
        model = TPMamba2ForCausalLM(full, TPContext(group=tp_group))
        for layer in full.layers:      # the unsharded mixers are no longer needed
            layer.mixer = None
        del full
        torch.cuda.empty_cache()
        engine = TPDPEngine(model, tp_group, dp_group, **kw)
        parallelism = f"tp{args.tp}xdp{dp}"
    elif args.ep and world > 1:
        from sneppx_alg_b200.models.deepseek import DeepSeekV2ForCausalLM
        model = DeepSeekV2ForCausalLM(cfg, dtype=torch.bfloat16, device=dev, ep_group=dist.group.WORLD)
        engine = make_engine(model, zero_stage=1, **kw)
        parallelism = f"ep{world}+zero1"
    else:
        model = build_model(cfg, dtype=torch.bfloat16, device=dev)
        if args.param_slots and world > 1:
            kw["param_slots"] = args.param_slots
        engine = make_engine(model, zero_stage=args.zero_stage, **kw)
        parallelism = f"zero{args.zero_stage}-dp{world}" + (f"-paramslots{args.param_slots}" if kw.get("param_slots") else "")

    def step(ids):
        return engine.step(ids, ids)

    res = measure(args, world, rank, local_rank, dev, step, V, B, S, 100 + dp_rank,
                  launches=lambda: _lib.launch_count, check=check_status, drain=getattr(engine, "finish", None))
    if args.ep and world > 1:
        from sneppx_alg_b200.parallel import expert as _ep
        d = torch.tensor([float(_ep.dropped_entries())], device=dev, dtype=torch.float64)
        dist.all_reduce(d)
        n_moe = sum(1 for m in model.modules() if hasattr(m, "ep_group") and hasattr(m, "router"))
        routed = float(B * S * world) * cfg.num_experts_per_token * max(n_moe, 1) * (args.warmup + 2 * args.steps)
        extra["expert_parallel"] = {"policy": _ep.policy_name(), "experts": _ep.expert_dtype_name(model),
                                    "dropped_fraction_of_routed_entries": float(d.item()) / routed}
    if rank == 0:
        print(json.dumps(result_line(args, world, dp, res, B, S, "ours", model_label(cfg, args), parallelism,
                                     res["launches"], extra)))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

#!/usr/bin/env python
"""Headline benchmark: training tokens/s of the Llama-3-8B-shape decoder (bf16, ZeRO-3 data parallel,
seq 4096, micro-batch 1 per GPU, AdamW beta 0.9/0.95 wd 0.1), synthetic token ids, random-init weights.

    python bench.py --gpus N --steps K --warmup W          # N > 1: launched by torch.distributed.run
    python bench.py --impl reference ...                    # the unmodified reference, if it can run this config

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
    """The reference's own code path. Its CUDA/NCCL layers do not build and its Python API is NumPy on
    CPU with no working Transformer backward, so the named config cannot run; say so and exit 0."""
    ref_dir = os.path.join(REPO, "baseline", "_ref")
    why = None
    if not os.path.isdir(os.path.join(ref_dir, "SneppX_ALG")):
        why = "reference not installed under baseline/_ref (offline pip install of the reference source tree not done on this box)"
    else:
        sys.path.insert(0, ref_dir)
        try:
            import SneppX_ALG  # noqa: F401
            why = ("reference installs but cannot run this config: its Python API is NumPy-on-CPU only (no GPU "
                   "execution, collectives are identity stubs) and backward through its Transformer raises a "
                   "matmul shape error; its CUDA/NCCL C layers do not compile")
        except Exception as e:  # noqa: BLE001
            why = f"reference import failed: {type(e).__name__}: {e}"
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def run_library(args):
    """The same step stated with PyTorch library ops only (cuBLAS through nn.functional.linear, SDPA attention,
    F.rms_norm, F.cross_entropy, NCCL reduce-scatter / all-gather over flat buffers, torch's fused AdamW on fp32 master
    shards): the comparator this repository can actually run on the box, since the reference cannot run the config.
    Same model shape, dtype recipe (bf16 weights / activations / gradients, fp32 master + moments), clipping and
    timing rules as the main arm; none of this repository's kernels are on the path."""
    import math

    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    from sneppx_alg_b200.models import config_from_name
    cfg = config_from_name(args.model)
    if cfg.architecture != "transformer":
        print(json.dumps({"impl": "library", "unavailable": "library arm covers the dense decoder config only"}))
        return 0
    L = args.layers or cfg.num_hidden_layers
    d, H, Hk, D, Fd, V = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, \
        cfg.intermediate_size, cfg.vocab_size
    torch.manual_seed(1234)
    shapes = [("emb", (V, d))]
    for i in range(L):
        shapes += [(f"{i}.n1", (d,)), (f"{i}.qkv", ((H + 2 * Hk) * D, d)), (f"{i}.o", (d, H * D)), (f"{i}.n2", (d,)),
                   (f"{i}.gu", (2 * Fd, d)), (f"{i}.down", (d, Fd))]
    shapes += [("nf", (d,)), ("head", (V, d))]
    unit = 256 * world
    offs, off = {}, 0
    for n, sh in shapes:
        offs[n] = off
        off += (math.prod(sh) + 255) // 256 * 256
    total = (off + unit - 1) // unit * unit
    flat = torch.empty(total, dtype=torch.bfloat16, device=dev)
    grad = torch.zeros(total, dtype=torch.bfloat16, device=dev)
    P = {}
    for n, sh in shapes:
        v = flat[offs[n]: offs[n] + math.prod(sh)].view(sh)
        if len(sh) == 1:
            v.fill_(1.0)
        else:
            v.normal_(0.0, 0.02)
        p = torch.nn.Parameter(v)
        p.grad = grad[offs[n]: offs[n] + math.prod(sh)].view(sh)
        P[n] = p
    if world > 1:
        dist.broadcast(flat, 0)
    sz = total // world
    master = flat[rank * sz: (rank + 1) * sz].float()
    CH = 1 << 28
    chunks = []
    for c0 in range(0, sz, CH):
        mp = torch.nn.Parameter(master[c0: c0 + CH])
        chunks.append((c0, mp, torch.optim.AdamW([mp], lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, fused=True)))
    gshard = torch.empty(sz, dtype=torch.bfloat16, device=dev) if world > 1 else None
    S = args.seq
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2, device=dev, dtype=torch.float32) / D))
    ang = torch.outer(torch.arange(S, device=dev, dtype=torch.float32), inv)
    cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]

    def rope(x):
        x1, x2 = x[..., : D // 2].float(), x[..., D // 2:].float()
        return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), -1).to(x.dtype)

    def forward_loss(ids):
        B = ids.shape[0]
        x = F.embedding(ids, P["emb"])
        for i in range(L):
            h = F.rms_norm(x, (d,), P[f"{i}.n1"], cfg.rms_norm_eps)
            qkv = F.linear(h, P[f"{i}.qkv"])
            q = rope(qkv[..., : H * D].view(B, S, H, D)).transpose(1, 2)
            k = rope(qkv[..., H * D:(H + Hk) * D].view(B, S, Hk, D)).transpose(1, 2)
            v = qkv[..., (H + Hk) * D:].view(B, S, Hk, D).transpose(1, 2)
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
            x = x + F.linear(a.transpose(1, 2).reshape(B, S, H * D), P[f"{i}.o"])
            h = F.rms_norm(x, (d,), P[f"{i}.n2"], cfg.rms_norm_eps)
            g, u = F.linear(h, P[f"{i}.gu"]).chunk(2, -1)
            x = x + F.linear(F.silu(g) * u, P[f"{i}.down"])
        x = F.rms_norm(x, (d,), P["nf"], cfg.rms_norm_eps)
        logits = F.linear(x[:, :-1], P["head"])
        return F.cross_entropy(logits.reshape(-1, V).float(), ids[:, 1:].reshape(-1))

    def step(ids):
        grad.zero_()
        loss = forward_loss(ids)
        loss.backward()
        if world > 1:
            dist.reduce_scatter_tensor(gshard, grad, op=dist.ReduceOp.AVG)
            g = gshard
        else:
            g = grad
        ss = torch.linalg.vector_norm(g, dtype=torch.float32).pow(2)
        if world > 1:
            dist.all_reduce(ss)
        nrm = ss.sqrt()
        coef = torch.clamp(1.0 / (nrm + 1e-6), max=1.0)
        for c0, mp, opt in chunks:
            mp.grad = g[c0: c0 + CH].float() * coef
            opt.step()
            mp.grad = None
        flat[rank * sz: (rank + 1) * sz].copy_(master)
        if world > 1:
            dist.all_gather_into_tensor(flat, flat[rank * sz: (rank + 1) * sz].clone())
        return loss.detach()

    B = args.micro_batch
    gen = torch.Generator().manual_seed(100 + rank)
    n_batches = args.warmup + 2 * args.steps + 2
    host = [torch.randint(0, V, (B, S), generator=gen, dtype=torch.int64).pin_memory() for _ in range(n_batches)]
    devb = [h.to(dev, non_blocking=True) for h in host]

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    it = 0
    for _ in range(args.warmup):
        step(devb[it])
        it += 1
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step(devb[it])
        it += 1
    e1.record()
    sync()
    ms = e0.elapsed_time(e1)
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    last = 0.0
    for _ in range(args.steps):
        last = float(step(host[it].to(dev, non_blocking=True)).item())
        it += 1
    f1.record()
    sync()
    ms_e2e = f0.elapsed_time(f1)
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = t.tolist()
    tokens = B * S * world * args.steps
    if rank == 0:
        print(json.dumps({
            "metric": "train tokens/sec", "value": tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random-init weights",
            "impl": "library (PyTorch ops: cuBLAS, SDPA, NCCL, torch fused AdamW; none of this repository's kernels)",
            "config": {"model": "llama3-8b-shape" if not args.layers else f"llama3-8b-shape-{args.layers}L(debug, invalid)",
                       "global_batch": B * world, "seq_len": S, "parallelism": f"zero-dp{world} (flat reduce-scatter / all-gather)",
                       "optimizer": "AdamW b=(0.9,0.95) wd=0.1 fp32 master+moments, clip 1.0"},
            "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": B * S * 8, "d2h_bytes_per_step": 4, "last_loss": last},
            "gpu_launches": 0, "clocks": clocks}))
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

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from sneppx_alg_b200.models import config_from_name, build_model
    from sneppx_alg_b200.ops import _lib, check_status
    from sneppx_alg_b200.parallel.zero import make_engine

    cfg = config_from_name(args.model)
    if args.layers:
        cfg.num_hidden_layers = cfg.num_layers = args.layers
    cfg.max_position_embeddings = max(args.seq, 8)
    torch.manual_seed(1234)
    if args.ep and world > 1:
        from sneppx_alg_b200.models.deepseek import DeepSeekV2ForCausalLM
        model = DeepSeekV2ForCausalLM(cfg, dtype=torch.bfloat16, device=dev, ep_group=dist.group.WORLD)
        stage = 1
    else:
        model = build_model(cfg, dtype=torch.bfloat16, device=dev)
        stage = args.zero_stage
    engine = make_engine(model, zero_stage=stage, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1,
                         max_grad_norm=1.0)
    B, S, V = args.micro_batch, args.seq, cfg.vocab_size
    gen = torch.Generator().manual_seed(100 + rank)
    n_batches = args.warmup + 2 * args.steps + 2
    host = [torch.randint(0, V, (B, S), generator=gen, dtype=torch.int64).pin_memory() for _ in range(n_batches)]
    dev_batches = [h.to(dev, non_blocking=True) for h in host]
    torch.cuda.synchronize()

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    it = 0
    for _ in range(args.warmup):
        engine.step(dev_batches[it], dev_batches[it])
        it += 1
    check_status()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # ---- device-timed region: inputs resident on the device
    launches0 = _lib.launch_count
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = engine.step(dev_batches[it], dev_batches[it])
        it += 1
    e1.record()
    sync()
    ms = e0.elapsed_time(e1)
    launches = _lib.launch_count - launches0
    # ---- end-to-end region: pinned host batch -> device every step, loss read back every step
    sync()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    last = 0.0
    for _ in range(args.steps):
        ids = host[it].to(dev, non_blocking=True)
        last = float(engine.step(ids, ids).item())
        it += 1
    f1.record()
    sync()
    ms_e2e = f0.elapsed_time(f1)
    clocks = sampler.stop() if rank == 0 else None
    check_status()
    t = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = t.tolist()
    tokens = B * S * world * args.steps
    ep_note = None
    if args.ep and world > 1:
        # capacity-factor expert parallelism: report how many routed (token, expert) entries were over capacity
        from sneppx_alg_b200.parallel import expert as _ep
        d = torch.tensor([float(_ep.dropped_entries())], device=dev, dtype=torch.float64)
        dist.all_reduce(d)
        n_moe = sum(1 for m in model.modules() if hasattr(m, "ep_group") and hasattr(m, "router"))
        routed = float(B * S * world) * cfg.num_experts_per_token * max(n_moe, 1) * (args.warmup + 2 * args.steps)
        ep_note = {"capacity_factor": float(os.environ.get("SX_EP_CAPACITY", "2.0")),
                   "dropped_fraction_of_routed_entries": float(d.item()) / routed}
    value = tokens / (ms / 1e3)
    e2e = tokens / (ms_e2e / 1e3)
    if rank == 0:
        line = {
            "metric": "train tokens/sec", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random-init weights",
            "impl": "ours",
            "config": {"model": (f"{cfg.name}-shape" if not args.layers else f"{cfg.name}-shape-{args.layers}L(debug, invalid)")
                       .replace("llama3-8B", "llama3-8b"),
                       "global_batch": B * world, "seq_len": S,
                       "parallelism": (f"ep{world}+zero1" if (args.ep and world > 1) else f"zero{stage}-dp{world}"),
                       "optimizer": "AdamW b=(0.9,0.95) wd=0.1 fp32 master+moments",
                       "l2": "per-step working set (>= 16 GB of weights) far exceeds the 126 MB L2"},
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": B * S * 8, "d2h_bytes_per_step": 4, "last_loss": last},
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if ep_note:
            line["config"]["expert_parallel"] = ep_note
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

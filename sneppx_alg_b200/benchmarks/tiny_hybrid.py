"""The CPU parity configuration: tiny HSS + SER hybrid (vocab 32000, d_model 256, 4 layers of RMSNorm -> Mamba-2 block
-> RMSNorm -> SER MoE with 8 SwiGLU experts top-2, tied embeddings), fp32, batch 2 x seq 512, forward + backward + AdamW
(lr 1e-3), seed 0.

``python -m sneppx_alg_b200.benchmarks.tiny_hybrid [--device cpu|cuda] [--steps N] [--out file.json]``

Reports the loss trajectory (it must fall from about ln(32000) = 10.37) and the step time. The reference's pieces of
this configuration are its C HSS and SER cores (dense-A LTI scan, biased MLP experts); their forward-only timings on
an 8-vCPU Xeon (2.7 GHz, gcc -O3, one thread) are the closest published comparison (HSS forward seq 512, 6 layers: 186.7 ms; SER forward 128 tokens,
32 experts: 21.5 ms) and there is no reference training step for this model.
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import torch


def run(device="cpu", steps=5, warmup=1, batch=2, seq=512):
    from ..models import create_model
    dev = torch.device(device)
    torch.manual_seed(0)
    dtype = torch.float32 if dev.type == "cpu" else torch.bfloat16
    model = create_model("hss-ser-tiny", dtype=dtype, device=dev)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, model.config.vocab_size, (batch, seq), generator=g).to(dev)
    sync = torch.cuda.synchronize if dev.type == "cuda" else (lambda: None)
    losses, times = [], []
    for s in range(warmup + steps):
        sync()
        t0 = time.perf_counter()
        out = model(ids, labels=ids)
        opt.zero_grad(set_to_none=True)
        out["loss"].backward()
        opt.step()
        sync()
        if s >= warmup:
            times.append((time.perf_counter() - t0) * 1e3)
        losses.append(float(out["ce_loss"]))
    n_params = sum(p.numel() for p in model.parameters())
    return {"config": "hss-ser-tiny", "device": str(dev), "dtype": str(dtype).replace("torch.", ""), "batch": batch, "seq": seq,
            "params": n_params, "ms_per_step": sum(times) / len(times), "min_ms": min(times),
            "tokens_per_s": batch * seq / (sum(times) / len(times) / 1e3), "ce_loss": losses}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    r = run(a.device, a.steps)
    print(json.dumps(r))
    if a.out:
        json.dump(r, open(a.out, "w"), indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())

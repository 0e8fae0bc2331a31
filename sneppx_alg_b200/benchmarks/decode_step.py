"""One decode step of the paged serving runner in isolation: ``--batch`` sequences that already hold ``--context``
tokens in the KV block pool (random contents; no prefill is run), one new token each.

``python -m sneppx_alg_b200.benchmarks.decode_step [--model llama3-8b] [--batch 64] [--context 2304] [--steps 20]
[--no-graphs] [--profile-one] [--out file.json]``

Reports the device time per step (CUDA events around ``--steps`` steps after 3 warm-up steps, the host preparing each
step as the engine does), the bytes a step must read (weights once, the KV of every sequence once) and the fraction of
the measured copy bandwidth that this is. ``--profile-one`` brackets a single eager step with
``cudaProfilerStart/Stop`` so that a profiler started with ``--profile-from-start off`` lists exactly the launches of
one step. The KV cache written here is larger than L2 many times over, and so are the weights.
"""
from __future__ import annotations

import argparse
import json

import torch


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--context", type=int, default=2304)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--profile-one", action="store_true")
    ap.add_argument("--out")
    a = ap.parse_args(argv)
    from ..models import create_model
    from ..serving.kv_cache import PagedKVCache
    from ..serving.llm_engine import LlamaPagedRunner
    from .kernels import _peaks
    dev = torch.device("cuda")
    torch.manual_seed(0)
    model = create_model(a.model, dtype=torch.bfloat16, device=dev).eval()
    cfg = model.config
    total = a.context + a.steps + 16
    cfg.max_position_embeddings = max(cfg.max_position_embeddings, total)
    bs = a.block_size
    per_seq = (total + bs - 1) // bs
    cache = PagedKVCache(cfg.num_hidden_layers, a.batch * per_seq + 8, bs, cfg.num_key_value_heads, cfg.head_dim,
                         device=dev, enable_prefix_cache=False)
    for k, v in zip(cache.k, cache.v):
        k.normal_()
        v.normal_()
    runner = LlamaPagedRunner(model, cache)
    if not a.no_graphs:
        runner.enable_graphs(a.batch, total)
    seqs = list(range(a.batch))
    for s in seqs:
        cache.add_sequence(s)
        cache.reserve(s, a.context)     # blocks for the context; their contents are the random fill above
    toks = [1 + (s % 100) for s in seqs]

    def step():
        return runner.decode(seqs, toks)      # reserves one more slot per sequence

    with torch.no_grad():
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        if a.profile_one:
            saved, runner._graphs = getattr(runner, "_graphs", None), None
            torch.cuda.profiler.start()
            step()
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
            runner._graphs = saved
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.steps):
            logits = step()
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.steps
    from .. import ops
    ops.check_status()
    wbytes = sum(p.numel() * p.element_size() for p in model.parameters())
    emb = model.embedding.weight
    if model.head_weight().data_ptr() != emb.data_ptr():
        wbytes -= emb.numel() * emb.element_size()      # the embedding table is gathered, not streamed
    ctx = a.context + 3 + a.steps // 2
    kvbytes = 2 * cfg.num_hidden_layers * a.batch * ctx * cfg.num_key_value_heads * cfg.head_dim * 2
    hbm, _, src = _peaks()
    r = {"case": "decode_step", "model": a.model, "batch": a.batch, "context": a.context, "graphs": not a.no_graphs,
         "ms_per_step": ms, "tokens_per_s": a.batch / ms * 1e3, "weight_bytes": wbytes, "kv_bytes": kvbytes,
         "gbs": (wbytes + kvbytes) / ms / 1e6, f"frac_hbm_of_{src}": (wbytes + kvbytes) / ms / 1e6 / hbm,
         "finite": bool(torch.isfinite(logits).all())}
    print(json.dumps(r))
    if a.out:
        with open(a.out, "w") as f:
            json.dump(r, f)
    return r


if __name__ == "__main__":
    main()

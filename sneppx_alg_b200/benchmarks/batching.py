"""Static against continuous batching on the same requests (the reference's ``benchmarks/serving_benchmark.py``
compares the two on a dummy model; here both drive a real model with a KV cache).

Static batching takes the requests in arrival order in groups of ``max_batch``, pads every group to its longest
prompt and decodes the whole group until its longest request is done, so short requests hold their slot idle.
Continuous batching (``LLMEngine``) lets a finished request's slot go to the next waiting one between steps. The
figures reported: decode steps, slot-steps spent on requests that had already finished, generated tokens per second.

    python -m sneppx_alg_b200.benchmarks.batching                 # tiny model on the CPU, or on the GPU when present
    python -m sneppx_alg_b200.benchmarks.batching --model llama3-8b --requests 128 --max-batch 32
"""
from __future__ import annotations

import argparse
import json
import time
from typing import Dict, List

import torch

from ..models import ModelConfig, build_model
from ..models.config import config_from_name
from ..serving.llm_engine import LLMEngine, SamplingParams


def make_requests(n: int, vocab: int, prompt_len=(4, 24), new_tokens=(2, 48), seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    reqs = []
    for _ in range(n):
        pl = int(torch.randint(prompt_len[0], prompt_len[1] + 1, (1,), generator=g))
        nt = int(torch.randint(new_tokens[0], new_tokens[1] + 1, (1,), generator=g))
        reqs.append((torch.randint(1, vocab, (pl,), generator=g).tolist(), nt))
    return reqs


@torch.no_grad()
def run_static(model, requests, max_batch: int) -> Dict[str, float]:
    """Groups of ``max_batch`` in arrival order, left-padded to one length, decoded in lock step to the group's
    longest output. Left padding keeps the last prompt token in the last position. The pad tokens are attended like
    any other token: this arm measures steps and time of the lock-step schedule, not the text it would produce."""
    dev = next(model.parameters()).device
    steps = idle = tokens = 0
    t0 = time.perf_counter()
    for s in range(0, len(requests), max_batch):
        group = requests[s:s + max_batch]
        width = max(len(p) for p, _ in group)
        longest = max(n for _, n in group)
        ids = torch.zeros(len(group), width, dtype=torch.long, device=dev)
        for i, (p, _) in enumerate(group):
            ids[i, width - len(p):] = torch.tensor(p, device=dev)
        out = model(ids, use_cache=True)
        cache, nxt = out["past_key_values"], out["logits"][:, -1].argmax(-1, keepdim=True)
        for step in range(longest):
            steps += 1
            idle += sum(1 for _, n in group if n <= step)
            tokens += sum(1 for _, n in group if n > step)
            if step + 1 < longest:
                nxt = model(nxt, past_key_values=cache, use_cache=True)["logits"][:, -1].argmax(-1, keepdim=True)
    if dev.type == "cuda":
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    return {"decode_steps": steps, "idle_slot_steps": idle, "generated_tokens": tokens, "seconds": dt, "tokens_per_s": tokens / dt}


def run_continuous(model, requests, max_batch: int, num_blocks: int = 1024, block_size: int = 16) -> Dict[str, float]:
    eng = LLMEngine(model, num_blocks=num_blocks, block_size=block_size, max_batch_size=max_batch, enable_prefix_cache=False)
    t0 = time.perf_counter()
    for p, n in requests:
        eng.submit(p, SamplingParams(max_new_tokens=n))
    eng.run_until_done()
    if next(model.parameters()).is_cuda:
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    tokens = sum(len(r.output) for r in eng.finished.values())
    return {"decode_steps": eng.stats["steps"], "idle_slot_steps": 0, "generated_tokens": tokens, "seconds": dt,
            "tokens_per_s": tokens / dt}


def compare(model, requests, max_batch: int) -> Dict[str, Dict[str, float]]:
    static = run_static(model, requests, max_batch)
    cont = run_continuous(model, requests, max_batch)
    return {"static": static, "continuous": cont,
            "step_ratio": static["decode_steps"] / max(1, cont["decode_steps"]),
            "throughput_ratio": cont["tokens_per_s"] / static["tokens_per_s"]}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", default="tiny")
    ap.add_argument("--requests", type=int, default=48)
    ap.add_argument("--max-batch", type=int, default=8)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    if a.model == "tiny":
        cfg = ModelConfig(hidden_size=256 if dev == "cuda" else 64, num_hidden_layers=2, num_attention_heads=2 if dev == "cuda" else 4,
                          num_key_value_heads=1 if dev == "cuda" else 2, intermediate_size=512 if dev == "cuda" else 128,
                          vocab_size=512, max_position_embeddings=256, rms_norm_eps=1e-5)
    else:
        cfg = config_from_name(a.model)
    model = build_model(cfg, dtype=torch.bfloat16 if dev == "cuda" else torch.float32, device=dev).eval()
    res = compare(model, make_requests(a.requests, cfg.vocab_size, seed=a.seed), a.max_batch)
    print(json.dumps({"model": a.model, "requests": a.requests, "max_batch": a.max_batch, **res}))
    return res


if __name__ == "__main__":
    main()

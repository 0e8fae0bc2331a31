"""Token sampling and whole-sequence generation loops: greedy, temperature / top-k / top-p sampling with repetition
penalty, beam search, lock-step batch generation. Function names and the model contract
``forward(input_ids, ..., past_key_values, use_cache) -> {"logits", "past_key_values"}`` follow the reference
(interface_bindings/generation.py:38-584; C twin kernel/inference/inference_engine.c:109-198)."""
from __future__ import annotations

from typing import List, Optional

import torch


def apply_repetition_penalty(logits, generated, penalty: float):
    if penalty == 1.0 or generated is None or generated.numel() == 0:
        return logits
    score = logits.gather(-1, generated)
    score = torch.where(score < 0, score * penalty, score / penalty)
    return logits.scatter(-1, generated, score)


def top_k_top_p_filtering(logits, top_k: int = 0, top_p: float = 1.0, filter_value: float = float("-inf")):
    if top_k and top_k > 0:
        kth = torch.topk(logits, min(top_k, logits.shape[-1]), dim=-1).values[..., -1:]
        logits = torch.where(logits < kth, torch.full_like(logits, filter_value), logits)
    if top_p < 1.0:
        sorted_logits, idx = torch.sort(logits, descending=True, dim=-1)
        probs = torch.softmax(sorted_logits, dim=-1)
        cum = probs.cumsum(-1)
        remove = cum - probs > top_p
        sorted_logits = sorted_logits.masked_fill(remove, filter_value)
        logits = torch.full_like(logits, filter_value).scatter(-1, idx, sorted_logits)
    return logits


def sample_from_logits(logits, do_sample=False, temperature=1.0, top_k=0, top_p=1.0, generator=None):
    """logits [B, V] -> token ids [B]."""
    if not do_sample or temperature <= 0:
        return logits.argmax(-1)
    logits = top_k_top_p_filtering(logits.float() / max(temperature, 1e-5), top_k, top_p)
    return torch.multinomial(torch.softmax(logits, -1), 1, generator=generator).squeeze(-1)


@torch.no_grad()
def generate(model, input_ids, max_new_tokens=32, do_sample=False, temperature=1.0, top_k=0, top_p=1.0,
             repetition_penalty=1.0, num_beams=1, eos_token_id: Optional[int] = None, generator=None):
    """Cached auto-regressive generation for one batch of equal-length prompts."""
    if num_beams > 1:
        return beam_search(model, input_ids, max_new_tokens, num_beams, eos_token_id)
    out = model(input_ids, use_cache=True)
    cache = out["past_key_values"]
    seq = input_ids
    done = torch.zeros(input_ids.shape[0], dtype=torch.bool, device=input_ids.device)
    for _ in range(max_new_tokens):
        logits = out["logits"][:, -1].float()
        logits = apply_repetition_penalty(logits, seq, repetition_penalty)
        nxt = sample_from_logits(logits, do_sample, temperature, top_k, top_p, generator)
        if eos_token_id is not None:
            nxt = torch.where(done, torch.full_like(nxt, eos_token_id), nxt)
            done |= nxt == eos_token_id
        seq = torch.cat([seq, nxt[:, None]], dim=1)
        if eos_token_id is not None and bool(done.all()):
            break
        out = model(nxt[:, None], past_key_values=cache, use_cache=True)
    return seq


greedy_search = lambda model, ids, max_new_tokens=32, **kw: generate(model, ids, max_new_tokens, **kw)  # noqa: E731


def sample_generation(model, ids, max_new_tokens=32, **kw):
    return generate(model, ids, max_new_tokens, do_sample=True, **kw)


@torch.no_grad()
def beam_search(model, input_ids, max_new_tokens=32, num_beams=4, eos_token_id=None, length_penalty=1.0):
    """Beam search without cache sharing tricks: beams are rows of the batch and the prefix is re-scored each step
    (clarity over speed; serving uses sampling/greedy through the paged engine)."""
    B = input_ids.shape[0]
    assert B == 1, "beam search takes one prompt"
    beams = [(input_ids[0], 0.0, False)]
    for _ in range(max_new_tokens):
        cand = []
        alive = [b for b in beams if not b[2]]
        if not alive:
            break
        batch = torch.stack([b[0] for b in alive])
        logp = torch.log_softmax(model(batch)["logits"][:, -1].float(), -1)
        top = torch.topk(logp, num_beams, dim=-1)
        for (seq, score, _), vals, idxs in zip(alive, top.values, top.indices):
            for v, i in zip(vals.tolist(), idxs.tolist()):
                cand.append((torch.cat([seq, seq.new_tensor([i])]), score + v, eos_token_id is not None and i == eos_token_id))
        cand += [b for b in beams if b[2]]
        cand.sort(key=lambda c: c[1] / (len(c[0]) ** length_penalty), reverse=True)
        beams = cand[:num_beams]
    return beams[0][0][None]


@torch.no_grad()
def batch_generate(model, prompts: List[torch.Tensor], max_new_tokens=32, pad_token_id=0, **kw):
    """Prompts of different lengths: grouped by length and generated group by group (exact, no padding effects)."""
    order = sorted(range(len(prompts)), key=lambda i: len(prompts[i]))
    results: List[Optional[torch.Tensor]] = [None] * len(prompts)
    i = 0
    while i < len(order):
        j = i
        while j < len(order) and len(prompts[order[j]]) == len(prompts[order[i]]):
            j += 1
        ids = torch.stack([prompts[k] for k in order[i:j]])
        out = generate(model, ids, max_new_tokens, **kw)
        for k, row in zip(order[i:j], out):
            results[k] = row
        i = j
    return results


def make_stop_fn(tokenizer, stop_strings, window: int = 64):
    """Stop predicate for ``SamplingParams.stop_fn``: true once the decoded tail of the output contains one of
    `stop_strings` (only the last `window` tokens are decoded each step)."""
    stops = [s for s in (stop_strings or []) if s]
    if not stops:
        return None
    return lambda out: any(s in tokenizer.decode(out[-window:]) for s in stops)


def truncate_at_stop(text: str, stop_strings) -> str:
    """Cuts `text` before the earliest occurrence of any stop string (the reference's generate() does the same
    after decoding, generation.py:244-534)."""
    cut = min((text.find(s) for s in (stop_strings or []) if s and s in text), default=-1)
    return text if cut < 0 else text[:cut]

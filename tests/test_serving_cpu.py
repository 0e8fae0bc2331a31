"""Paged continuous-batching engine against plain cached generation (CPU, fp32): same greedy tokens, prefix cache
hits, copy-on-write, sampling utilities."""
import torch

from sneppx_alg_b200.models import ModelConfig, build_model
from sneppx_alg_b200.serving.generation import (apply_repetition_penalty, batch_generate, generate,
                                               top_k_top_p_filtering)
from sneppx_alg_b200.serving.kv_cache import KVBlockPool, PagedKVCache
from sneppx_alg_b200.serving.llm_engine import LLMEngine, SamplingParams


def _model():
    torch.manual_seed(0)
    cfg = ModelConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                      intermediate_size=128, vocab_size=97, max_position_embeddings=128, rms_norm_eps=1e-5)
    return build_model(cfg).eval()


def test_engine_matches_cached_generation_and_reuses_prefix():
    model = _model()
    g = torch.Generator().manual_seed(1)
    shared = torch.randint(0, 97, (20,), generator=g).tolist()
    prompts = [shared + torch.randint(0, 97, (n,), generator=g).tolist() for n in (3, 9, 5)]
    ref = [generate(model, torch.tensor([p]), max_new_tokens=8)[0, len(p):].tolist() for p in prompts]
    eng = LLMEngine(model, num_blocks=64, block_size=4, max_batch_size=2)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=8))
    assert outs == ref
    assert eng.cache.pool.num_free + len(eng.cache.prefix.table) == 64      # everything returned except cached blocks
    # a second wave with the same prefix is served from the prefix cache and still matches
    outs2 = eng.generate(prompts[:1], SamplingParams(max_new_tokens=8))
    assert outs2[0] == ref[0] and eng.stats["cached_prefix_tokens"] >= 20


def test_block_pool_refcount_and_cow():
    pool = KVBlockPool(4)
    a = pool.allocate()
    pool.share(a)
    pool.release(a)
    assert pool.num_free == 3
    pool.release(a)
    assert pool.num_free == 4
    cache = PagedKVCache(1, 8, 2, 1, 4, dtype=torch.float32, device="cpu", enable_prefix_cache=False)
    cache.add_sequence(0)
    cache.reserve(0, 3)
    cache.k[0][cache.tables[0][1]].fill_(7.0)
    cache.fork(0, 1)
    slots = cache.reserve(1, 1)            # writes into the shared, half-full block -> copy
    assert cache.tables[1][1] != cache.tables[0][1]
    assert float(cache.k[0][cache.tables[1][1]][0, 0, 0]) == 7.0 and slots[0] == cache.tables[1][1] * 2 + 1


def test_sampling_filters():
    logits = torch.tensor([[1.0, 2.0, 3.0, 4.0]])
    f = top_k_top_p_filtering(logits.clone(), top_k=2)
    assert torch.isinf(f[0, :2]).all() and not torch.isinf(f[0, 2:]).any()
    f = top_k_top_p_filtering(logits.clone(), top_p=0.6)
    assert not torch.isinf(f[0, 3]) and torch.isinf(f[0, 0])
    p = apply_repetition_penalty(torch.tensor([[2.0, -2.0]]), torch.tensor([[0, 1]]), 2.0)
    assert p.tolist() == [[1.0, -4.0]]
    model = _model()
    outs = batch_generate(model, [torch.tensor([1, 2, 3]), torch.tensor([4, 5])], max_new_tokens=3)
    assert len(outs[0]) == 6 and len(outs[1]) == 5


def test_engine_serves_recurrent_state_models():
    """Mamba-2 through the continuous-batching engine: tokens equal the model's own greedy decoding from a full
    re-forward at every step, for requests of different lengths that join and leave the batch at different times."""
    import torch
    from sneppx_alg_b200.models import ModelConfig, build_model
    from sneppx_alg_b200.serving.llm_engine import LLMEngine, SamplingParams, StatefulRunner
    torch.manual_seed(0)
    cfg = ModelConfig(architecture="mamba2", hidden_size=32, num_hidden_layers=2, vocab_size=96, ssm_state_size=8,
                      ssm_conv_kernel=4, ssm_expand=2, ssm_head_dim=8, ssm_ngroups=1, ssm_chunk_size=8, rms_norm_eps=1e-5)
    model = build_model(cfg).eval()
    prompts = [[5, 9, 33, 2, 7], [11, 12], [70, 3, 3, 8, 1, 2, 90, 4, 6]]
    lens = [6, 3, 4]
    eng = LLMEngine(model, max_batch_size=2)   # two slots for three requests: the third joins when one finishes
    assert isinstance(eng.runner, StatefulRunner)
    ids = [eng.submit(p, SamplingParams(max_new_tokens=n)) for p, n in zip(prompts, lens)]
    eng.run_until_done()
    for rid, p, n in zip(ids, prompts, lens):
        seq = list(p)
        with torch.no_grad():
            for _ in range(n):
                seq.append(int(model(torch.tensor([seq]))["logits"][0, -1].argmax()))
        assert eng.finished[rid].output == seq[len(p):]
    assert eng.runner.states == {} and eng.cache.pool.num_free == 2


def test_same_length_prompts_share_one_prefill_pass():
    """Waiting requests whose prompts have the same length are prefilled as one batch (one pass over the weights);
    the tokens are those of one-by-one generation, the prompt of another length still goes alone, and the batch
    respects the token budget."""
    model = _model()
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 97, (12,), generator=g).tolist() for _ in range(5)] + [torch.randint(0, 97, (7,), generator=g).tolist()] + \
              [torch.randint(0, 97, (12,), generator=g).tolist() for _ in range(2)]
    ref = [generate(model, torch.tensor([p]), max_new_tokens=6)[0, len(p):].tolist() for p in prompts]
    eng = LLMEngine(model, num_blocks=128, block_size=4, max_batch_size=8, max_prefill_tokens=40, enable_prefix_cache=False)
    calls = []
    orig = eng.runner.prefill_batch
    eng.runner.prefill_batch = lambda ids, ps: (calls.append(len(ps)), orig(ids, ps))[1]
    out = eng.generate(prompts, SamplingParams(max_new_tokens=6))
    assert out == ref
    assert calls and calls[0] == 3                     # 40-token budget: three 12-token prompts per pass
    assert eng.stats["prefill_tokens"] == sum(len(p) for p in prompts)
    assert not eng.cache.tables and eng.cache.pool.free_count() == 128 if hasattr(eng.cache.pool, "free_count") else True


def test_tensor_parallel_engine_matches_single_rank_tokens():
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    r = subprocess.run([sys.executable, os.path.join(here, "mp_tp_serving_check.py"), "2", str(29820 + os.getpid() % 9)],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "TP_SERVING_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_tensor_parallel_serving_over_http_matches_single_rank_tokens():
    """Rank 0 serves POST /v1/generate, rank 1 mirrors it (requests broadcast once per engine step)."""
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    r = subprocess.run([sys.executable, os.path.join(here, "mp_tp_http_check.py"), "2", str(29840 + os.getpid() % 9)],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "TP_HTTP_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_prefix_cache_gives_blocks_back_under_pressure():
    """A pool mostly pinned by cached prefixes must still admit new requests (entries nobody shares are evicted,
    least recently used first), never run dry in the middle of a generation, and fail a request that can never
    fit instead of spinning."""
    model = _model()
    g = torch.Generator().manual_seed(3)
    eng = LLMEngine(model, num_blocks=24, block_size=4, max_batch_size=4)
    assert eng.cache.prefix.max_entries <= 12          # capped at a fraction of the pool
    ref_prompts = [torch.randint(0, 97, (17 + i,), generator=g).tolist() for i in range(8)]
    refs = [generate(model, torch.tensor([p]), max_new_tokens=6)[0, len(p):].tolist() for p in ref_prompts]
    # eight different prompts of ~6 blocks each through a 24-block pool: the cache fills, then has to yield
    outs = eng.generate(ref_prompts, SamplingParams(max_new_tokens=6))
    assert outs == refs
    assert not eng.failed
    assert eng.cache.pool.num_free + len(eng.cache.prefix.table) == 24
    # a request larger than the whole pool is rejected at once; the engine goes idle instead of looping
    rid = eng.submit(list(range(90)) + [1] * 30, SamplingParams(max_new_tokens=8))
    done = eng.run_until_done(max_steps=50)
    assert rid in eng.failed and rid in done and not eng.has_work()
    # and the engine still serves afterwards
    assert eng.generate(ref_prompts[:1], SamplingParams(max_new_tokens=6))[0] == refs[0]

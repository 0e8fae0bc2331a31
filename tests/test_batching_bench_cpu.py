"""Static against continuous batching (``benchmarks/batching.py``) on a tiny CPU model: both generate the same number
of tokens; continuous batching needs fewer decode steps and wastes no slot on finished requests."""
import torch

from sneppx_alg_b200.benchmarks import batching
from sneppx_alg_b200.models import ModelConfig, build_model


def test_continuous_batching_needs_fewer_steps():
    torch.manual_seed(0)
    cfg = ModelConfig(hidden_size=32, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1, intermediate_size=64,
                      vocab_size=64, max_position_embeddings=128, rms_norm_eps=1e-5)
    model = build_model(cfg).eval()
    reqs = batching.make_requests(24, 64, prompt_len=(3, 10), new_tokens=(1, 30), seed=1)
    res = batching.compare(model, reqs, max_batch=4)
    want = sum(n for _, n in reqs)
    assert res["static"]["generated_tokens"] == res["continuous"]["generated_tokens"] == want
    assert res["static"]["idle_slot_steps"] > 0 and res["continuous"]["idle_slot_steps"] == 0
    # static: every group runs to its longest request
    groups = [reqs[i:i + 4] for i in range(0, 24, 4)]
    assert res["static"]["decode_steps"] == sum(max(n for _, n in g) for g in groups)
    assert res["continuous"]["decode_steps"] < res["static"]["decode_steps"] and res["step_ratio"] > 1.1
    out = batching.main(["--requests", "8", "--max-batch", "4"])
    assert out["continuous"]["generated_tokens"] == out["static"]["generated_tokens"]

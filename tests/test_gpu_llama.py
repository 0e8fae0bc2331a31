"""End-to-end: a small Llama-shape model trains through the flat-buffer engine on the native kernels and
tracks an fp32 PyTorch run of the same model."""
import copy

import pytest
import torch

from sneppx_alg_b200 import ops
from sneppx_alg_b200.models import ModelConfig, build_model
from sneppx_alg_b200.training.engine import TrainEngine

pytestmark = pytest.mark.gpu


def test_llama_step_matches_fp32_oracle():
    torch.manual_seed(0)
    cfg = ModelConfig(hidden_size=512, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                      intermediate_size=1024, vocab_size=2048, max_position_embeddings=256, rms_norm_eps=1e-5)
    ref = build_model(cfg)                       # fp32 on CPU: plain PyTorch path
    model = copy.deepcopy(ref).to("cuda", torch.bfloat16)
    ref_eng = TrainEngine(ref, lr=1e-3, weight_decay=0.1, max_grad_norm=1.0)
    eng = TrainEngine(model, lr=1e-3, weight_decay=0.1, max_grad_norm=1.0)
    losses, ref_losses = [], []
    for step in range(6):
        ids = torch.randint(0, cfg.vocab_size, (2, 256), generator=torch.Generator().manual_seed(step))
        ref_losses.append(ref_eng.step(ids, ids).item())
        losses.append(eng.step(ids.cuda(), ids.cuda()).item())
    ops.check_status()
    assert abs(losses[0] - ref_losses[0]) < 3e-2
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 0.1, (losses, ref_losses)
    # same batch repeated: the loss must go down
    ids = torch.randint(0, cfg.vocab_size, (2, 256), generator=torch.Generator().manual_seed(0)).cuda()
    first = eng.step(ids, ids).item()
    for _ in range(5):
        last = eng.step(ids, ids).item()
    assert last < first


def test_overlapped_optimizer_gives_the_same_parameters():
    """Per-bucket AdamW on a side stream (the next forward waits bucket by bucket) against the single-stream step:
    identical losses and bit-identical master weights after several steps."""
    torch.manual_seed(0)
    cfg = ModelConfig(hidden_size=512, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                      intermediate_size=1024, vocab_size=2048, max_position_embeddings=256, rms_norm_eps=1e-5)
    base = build_model(cfg).to("cuda", torch.bfloat16)
    a = TrainEngine(copy.deepcopy(base), lr=1e-3, weight_decay=0.1, max_grad_norm=1.0, overlap_optimizer=False)
    b = TrainEngine(copy.deepcopy(base), lr=1e-3, weight_decay=0.1, max_grad_norm=1.0, overlap_optimizer=True)
    assert b._opt_stream is not None and len(b._ranges) == cfg.num_hidden_layers + 2
    assert b._ranges[0][0] == 0 and b._ranges[-1][1] == b.fp.total
    assert all(x[1] == y[0] for x, y in zip(b._ranges, b._ranges[1:]))
    for step in range(5):
        ids = torch.randint(0, cfg.vocab_size, (2, 256), generator=torch.Generator().manual_seed(step)).cuda()
        la, lb = a.step(ids, ids), b.step(ids, ids)
        assert la.item() == lb.item()
    sa, sb = a.state_dict(), b.state_dict()     # state_dict waits for the updates in flight
    assert torch.equal(sa["master"], sb["master"]) and torch.equal(sa["m"], sb["m"]) and torch.equal(sa["v"], sb["v"])
    assert torch.equal(a.fp.flat, b.fp.flat)
    ops.check_status()


def test_llama_generate_cached_equals_uncached():
    torch.manual_seed(0)
    cfg = ModelConfig(hidden_size=256, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1,
                      intermediate_size=512, vocab_size=512, max_position_embeddings=256, rms_norm_eps=1e-5)
    model = build_model(cfg, dtype=torch.bfloat16, device="cuda").eval()
    ids = torch.randint(0, 512, (2, 40), device="cuda")
    with torch.no_grad():
        full = model(ids)["logits"]
        cache = model.init_kv_cache(2, 64)
        a = model(ids[:, :32], past_key_values=cache)["logits"]
        b = model(ids[:, 32:], past_key_values=cache)["logits"]
    ops.check_status()
    got = torch.cat([a, b], 1).float()
    assert (got - full.float()).abs().max().item() < 0.15

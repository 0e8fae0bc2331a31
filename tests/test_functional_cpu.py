"""CPU reference paths of ``ops.functional`` on inputs that are views (sliced, transposed): the fallbacks must not
assume contiguous memory."""
import torch

from sneppx_alg_b200 import ops
from sneppx_alg_b200.models import ModelConfig, build_model
from sneppx_alg_b200.training.engine import TrainEngine


def test_cross_entropy_accepts_sliced_targets_and_logits():
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(4, 9, 11, generator=g)
    ids = torch.randint(0, 11, (4, 10), generator=g)
    tgt = ids[:, 1:]                                                          # a non-contiguous view
    assert not tgt.is_contiguous()
    want = torch.nn.functional.cross_entropy(logits.reshape(-1, 11), tgt.reshape(-1))
    assert torch.allclose(ops.cross_entropy(logits, tgt), want)
    assert torch.allclose(ops.cross_entropy(logits.transpose(0, 1), tgt.transpose(0, 1)), want)
    h, w = torch.randn(4, 9, 6, generator=g), torch.randn(11, 6, generator=g)
    want2 = torch.nn.functional.cross_entropy((h @ w.T).reshape(-1, 11), tgt.reshape(-1))
    assert torch.allclose(ops.linear_cross_entropy(h, w, tgt), want2, atol=1e-6)


def test_train_engine_step_with_pre_shifted_views():
    torch.manual_seed(0)
    cfg = ModelConfig(hidden_size=32, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1,
                      intermediate_size=64, vocab_size=50, max_position_embeddings=32, rms_norm_eps=1e-5)
    eng = TrainEngine(build_model(cfg), lr=1e-2)
    ids = torch.randint(0, 50, (3, 12))
    a = float(eng.step(ids[:, :-1], ids[:, 1:], shift_labels=False))
    b = float(eng.step(ids[:, :-1], ids[:, 1:], shift_labels=False))
    assert a > b > 0

"""CPU behaviour of the auxiliary ops (the PyTorch restatements that the GPU tests use as oracles)."""
import torch

from sneppx_alg_b200.ops import aux


def test_philox_known_answer():
    # Random123 known-answer test for philox4x32-10: counter 0, key 0
    w = aux.philox_reference(0, 0, 1)[0].tolist()
    assert [hex(v) for v in w] == ["0x6627e8d5", "0xe169c58d", "0xbc57ac4c", "0x9b00dbd8"]


def test_rng_reference_statistics_and_streams():
    u = aux.rng_fill(100000, "uniform", -1.0, 3.0, seed=7, device="cpu")
    assert u.min() >= -1.0 and u.max() < 3.0 and abs(float(u.mean()) - 1.0) < 0.02
    z = aux.rng_fill(100000, "normal", 2.0, 0.5, seed=7, device="cpu")
    assert abs(float(z.mean()) - 2.0) < 0.01 and abs(float(z.std()) - 0.5) < 0.01
    b = aux.rng_fill(100000, "bernoulli", 0.3, seed=7, device="cpu")
    assert abs(float(b.mean()) - 0.3) < 0.01
    assert torch.equal(aux.rng_fill(1001, seed=3, device="cpu"), aux.rng_fill(1001, seed=3, device="cpu"))
    assert not torch.equal(aux.rng_fill(64, seed=3, offset=0, device="cpu"), aux.rng_fill(64, seed=3, offset=1, device="cpu"))


def test_dropout_cpu_mask_regenerated_in_backward():
    x = torch.randn(4, 64, requires_grad=True)
    y = aux.dropout(x, 0.25, seed=11, offset=2)
    keep = aux.dropout_mask_reference(256, 0.25, 11, 2).view(4, 64)
    assert torch.allclose(y, x * keep / 0.75) and 0.6 < keep.float().mean() < 0.9
    y.sum().backward()
    assert torch.allclose(x.grad, keep.float() / 0.75)
    assert aux.dropout(x, 0.25, seed=11, training=False) is x


def test_compression_references():
    x = torch.randn(1024)
    q, s = aux.quant_int8(x)
    assert q.dtype == torch.int8 and s.shape == (4,)
    assert (aux.dequant_int8(q, s) - x).abs().max() <= s.max() * 0.5001
    kept, res = aux.block_top2(x)
    assert torch.equal(kept + res, x) and int((kept.view(-1, 32) != 0).sum(1).max()) == 2
    assert torch.all(kept.view(-1, 32).abs().amax(1) == x.view(-1, 32).abs().amax(1))
    ties = torch.ones(32)
    k2, _ = aux.block_top2(ties)
    assert k2.nonzero().flatten().tolist() == [0, 1]
    avg = aux.weighted_average([torch.ones(8), 3 * torch.ones(8)], [0.25, 0.75])
    assert torch.allclose(avg, torch.full((8,), 2.5))


def test_arc_steps_reference():
    x0 = torch.full((8,), 0.5)
    g = torch.tensor([1.0, -1.0, 0.0, 2.0, -3.0, 0.5, -0.5, 0.0])
    adv = aux.arc_step("fgsm", x0, g, eps=0.1)
    assert torch.allclose(adv, 0.5 + 0.1 * torch.sign(g))
    cur = adv
    for _ in range(5):
        cur = aux.arc_step("pgd", cur, g, x0, eps=0.15, alpha=0.1)
    assert torch.all((cur - x0).abs() <= 0.15 + 1e-6) and torch.allclose(cur, 0.5 + 0.15 * torch.sign(g))
    assert torch.allclose(aux.arc_step("obfuscate", g, eps=0.01), g + 0.01 * torch.sin(100 * g))
    s = aux.arc_step("smooth", torch.zeros(4096), eps=0.2, seed=5)
    assert abs(float(s.std()) - 0.2) < 0.02


def test_fm_block_compression_and_average():
    from sneppx_alg_b200.algorithms import fm
    torch.manual_seed(0)
    g = torch.randn(3, 50)  # 150 values: four full blocks and a tail of 22
    kept, res = fm.compress_block_top2(g)
    assert torch.equal(kept + res, g) and int((kept.reshape(-1)[:128] != 0).sum()) == 8
    assert torch.equal(kept.reshape(-1)[128:], g.reshape(-1)[128:])
    ef = fm.BlockErrorFeedback()
    sent = sum(ef.compress(g) for _ in range(40))
    # error feedback: everything is sent eventually, up to the residual still held back
    assert torch.allclose(sent + ef.residual, 40 * g, atol=1e-4)
    q, s, n = fm.quantize_grad_int8(g)
    back = fm.dequantize_grad_int8(q, s, n, g.shape)
    assert back.shape == g.shape and (back - g).abs().max() <= s.max() * 0.5001
    avg = fm.federated_average([torch.zeros(4, 4), torch.ones(4, 4)], [1, 3])
    assert torch.allclose(avg, torch.full((4, 4), 0.75))


def test_arc_seeded_smoothing_is_reproducible():
    from sneppx_alg_b200.algorithms import arc
    x = torch.linspace(-1, 1, 64)
    a = arc.randomized_smoothing(lambda t: t * 2, x, sigma=0.1, samples=4, seed=3)
    b = arc.randomized_smoothing(lambda t: t * 2, x, sigma=0.1, samples=4, seed=3)
    assert torch.equal(a, b) and (a - 2 * x).abs().max() < 0.5

"""C++ host components: tokenizer, model factory, serving core, edge runtime, and the C++ oracles against the
PyTorch statements of the same ops (two independent implementations must agree)."""
import numpy as np
import torch

from sneppx_alg_b200.ops import moe, ssm
from sneppx_alg_b200.optim.fused import adamw_reference
from sneppx_alg_b200.utils import host


def test_bpe_tokenizer_roundtrip(tmp_path):
    text = "the quick brown fox jumps over the lazy dog. the fox, the dog, the end. " * 20
    tok = host.BPETokenizer()
    assert tok.train(text, 300) > 0 and tok.vocab_size <= 300
    ids = tok.encode("the quick fox — ünïcode")
    assert tok.decode(ids) == "the quick fox — ünïcode" and len(ids) < len("the quick fox — ünïcode".encode())
    tok.save(str(tmp_path / "tok.txt"))
    assert host.BPETokenizer().load(str(tmp_path / "tok.txt")).encode("the quick fox") == tok.encode("the quick fox")


def test_model_factory():
    c = host.factory_config("meta-llama/Llama-3-8B")
    assert c["hidden_size"] == 4096 and c["num_key_value_heads"] == 8 and 7.9e9 < c["num_parameters"] < 8.1e9
    assert host.factory_config("mistral-7b")["sliding_window"] == 4096
    e = host.factory_config("llama3-8b", extend_to=65536, method="ntk")
    assert e["max_position_embeddings"] == 65536 and e["rope_theta"] == 5e5 * 8
    assert "qwen2:72b" in host.factory_search("qwen")


def test_serving_core():
    sc = host.ServingCore(max_batch=3, timeout_ms=10000.0)
    for i, pr in enumerate((5, 1, 3, 1)):
        sc.submit(i, pr)
    assert sc.next_batch() == [1, 3, 2]          # full batch fires; priority then arrival order
    assert sc.next_batch() == [] and sc.next_batch(force=True) == [0]
    for i in range(100):
        sc.record(i / 100.0, ok=True)
    m = sc.metrics()
    assert 0.45 < m["p50"] < 0.55 and m["requests"] == 100
    assert host.ServingCore.route("abc", [0.0, 1.0]) == 1
    picks = {host.ServingCore.route(f"r{i}", [0.5, 0.5]) for i in range(50)}
    assert picks == {0, 1}
    sc.breaker_config(fail_threshold=2, cooldown_ms=50.0)
    sc.record(0.1, ok=False)
    sc.record(0.1, ok=False)
    assert not sc.breaker_allow()
    import time
    time.sleep(0.08)
    assert sc.breaker_allow()                    # half-open probe after the cool-down


def test_edge_runtime(tmp_path):
    rng = np.random.RandomState(0)
    w1, b1, w2 = rng.randn(8, 16).astype(np.float32), rng.randn(16).astype(np.float32), rng.randn(16, 4).astype(np.float32)
    p = str(tmp_path / "m.edge")
    host.write_edge_model(p, [("matmul", w1), ("bias", b1), ("relu",), ("matmul", w2)])
    x = rng.randn(5, 8).astype(np.float32)
    assert np.allclose(host.EdgeModel(p).run(x), np.maximum(x @ w1 + b1, 0) @ w2, atol=1e-4)


def test_cpp_oracles_agree_with_pytorch():
    torch.manual_seed(0)
    B, L, H, P, G, N = 2, 40, 4, 8, 2, 16
    x, dt = torch.randn(B, L, H, P), torch.rand(B, L, H) * 0.1 + 1e-3
    A, Bm, Cm, D = -torch.rand(H) * 3 - 0.5, torch.randn(B, L, G, N), torch.randn(B, L, G, N), torch.randn(H)
    y_cpp = host.oracle_ssd(*[t.numpy() for t in (x, dt, A, Bm, Cm, D)])
    assert np.allclose(y_cpp, ssm.ssd_reference(x, dt, A, Bm, Cm, D).numpy(), atol=1e-4)
    assert np.allclose(y_cpp, ssm.ssd_chunked(x, dt, A, Bm, Cm, D, chunk=16).numpy(), atol=1e-4)
    logits = torch.randn(50, 8)
    idx_cpp, w_cpp = host.oracle_router(logits.numpy(), 2)
    idx, w, _, _ = moe.route(logits, 2)
    assert np.array_equal(idx_cpp, idx.numpy()) and np.allclose(w_cpp, w.numpy(), atol=1e-6)
    p, g = torch.randn(100), torch.randn(100)
    m, v = torch.zeros(100), torch.zeros(100)
    pc, mc, vc = p.numpy().copy(), m.numpy().copy(), v.numpy().copy()
    for step in (1, 2, 3):
        adamw_reference(p, m, v, g, 1e-2, 0.9, 0.95, 1e-8, 0.1, step)
        host.oracle_adamw(pc, mc, vc, g.numpy(), 1e-2, 0.9, 0.95, 1e-8, 0.1, step)
    assert np.allclose(pc, p.numpy(), atol=1e-6)

"""Expression-graph fusion planner, jit transforms, storage / cache, registry, watermark, HF round trip."""
import torch

from sneppx_alg_b200 import jit
from sneppx_alg_b200 import tensor as T
from sneppx_alg_b200.graph import ExprGraph
from sneppx_alg_b200.hub import hf
from sneppx_alg_b200.models import create_model
from sneppx_alg_b200.serving.watermark import Watermark
from sneppx_alg_b200.utils.registry import EvalMonitor, ModelRegistry, PromptRegistry
from sneppx_alg_b200.utils.storage import CacheManager, open_storage


def test_expr_graph_fusion():
    torch.manual_seed(0)
    g = ExprGraph()
    x = g.input("x")
    w1, b1, w2 = g.const(torch.randn(16, 8)), g.const(torch.randn(16)), g.const(torch.randn(4, 16))
    h = g.unary("relu", g.add(g.matmul(x, w1), b1))
    y = g.unary("tanh", g.unary("neg", g.matmul(h, w2)))
    plan = g.plan_fusions([y])
    assert [p["kind"] for p in plan] == ["gemm_epilogue", "unary_chain"] and len(plan[0]["nodes"]) == 3
    xs = torch.randn(5, 8)
    fused = g.run([y], {"x": xs})[0]
    n_fused = g.launches
    plain = g.run([y], {"x": xs}, fuse=False)[0]
    assert torch.allclose(fused, plain, atol=1e-5) and n_fused == 3 and g.launches == 6
    shapes = {i: (5, 16) for i in range(len(g.nodes))}
    assert g.memory_estimate([y], shapes) < g.memory_estimate([y], shapes, fused=False)


def test_jit_and_tensor_api():
    f = lambda v: (v ** 3).sum()  # noqa: E731
    v = torch.tensor([1.0, 2.0])
    assert torch.allclose(jit.grad(f)(v), 3 * v ** 2)
    assert torch.allclose(jit.hessian(f)(v), torch.diag(6 * v))
    assert torch.allclose(jit.vmap(lambda r: r.sum())(torch.ones(3, 4)), torch.full((3,), 4.0))
    assert jit.jacobian(lambda r: r * 2)(v).shape == (2, 2)
    fn = lambda a: a + 1  # noqa: E731
    traced = jit.trace(fn, v)                             # CPU: a replayed tape, no CUDA-graph capture
    assert torch.equal(traced(v * 2), fn(v * 2)) and traced.traces == 1
    x = torch.tensor([0.113, -0.5], requires_grad=True)
    T.fake_quant(x, 4).sum().backward()
    assert torch.allclose(x.grad, torch.ones(2))           # straight-through


def test_storage_cache_registry(tmp_path):
    st = open_storage("s3://bucket", mirror_root=str(tmp_path))
    digest = st.put("a/b.bin", b"hello")
    assert st.get("a/b.bin") == b"hello" and len(digest) == 64 and st.list("a/") == ["a/b.bin"]
    assert st.url("a/b.bin") == "s3://bucket/a/b.bin"
    st.delete("a/b.bin")
    assert not st.exists("a/b.bin")
    c = CacheManager(10)
    c.put("x", b"12345")
    c.put("y", b"12345")
    assert c.get("x") == b"12345"
    c.put("z", b"123")                                     # evicts y (least recently used)
    assert c.get("y") is None and c.get("x") is not None and c.stats()["evictions"] == 1
    assert c.get("w", loader=lambda k: b"ww") == b"ww"
    reg = ModelRegistry(str(tmp_path / "reg.json"))
    v1 = reg.register("m", "file://m1", {"acc": 0.7}, ["base"])
    v2 = reg.register("m", "file://m2", {"acc": 0.8}, ["ft"], parent=f"m:{v1}")
    reg.transition("m", v1, "production")
    reg.transition("m", v2, "production")
    assert reg.get("m", stage="production")["version"] == 2 and reg.get("m", 1)["stage"] == "archived"
    assert reg.lineage("m", 2) == ["m:2", "m:1"]
    assert [r["version"] for r in ModelRegistry(str(tmp_path / "reg.json")).search("m", min_metric=("acc", 0.75))] == [2]
    pr = PromptRegistry()
    pr.register("qa", "Q: {q}\nA:")
    assert pr.render("qa", q="why") == "Q: why\nA:"
    mon = EvalMonitor(window=5, tolerance=0.1)
    assert not any(mon.observe(v) for v in (0.8, 0.81, 0.79, 0.8)) and mon.observe(0.6)


def test_watermark_detects():
    torch.manual_seed(0)
    wm = Watermark(200, gamma=0.5, delta=6.0)
    toks = [3]
    for _ in range(60):
        logits = wm.apply(torch.randn(1, 200), [toks[-1]])
        toks.append(int(torch.distributions.Categorical(logits=logits[0]).sample()))
    assert wm.detect(toks)["watermarked"]
    plain = torch.randint(0, 200, (61,)).tolist()
    assert not wm.detect(plain)["watermarked"]


def test_hf_round_trip(tmp_path):
    torch.manual_seed(0)
    m = create_model("llama3-tiny")
    hf.to_huggingface(m, str(tmp_path / "hf"))
    m2 = hf.from_huggingface(str(tmp_path / "hf"))
    ids = torch.randint(0, 512, (1, 9))
    assert torch.allclose(m(ids)["logits"], m2(ids)["logits"], atol=1e-5)
    out = hf.pipeline("text-generation", m2)("hi", max_new_tokens=3)
    assert isinstance(out[0]["generated_text"], str)


def test_vizmon_graph_and_dashboard_page():
    import json
    import urllib.request

    import torch
    from sneppx_alg_b200.utils.vizmon import VizMon
    v = VizMon()
    for i in range(4):
        v.scalar("loss", 5.0 - i)
    v.graph_from_module(torch.nn.Sequential(torch.nn.Linear(2, 3), torch.nn.ReLU()))
    port = v.serve()
    try:
        g = json.load(urllib.request.urlopen(f"http://127.0.0.1:{port}/graph.json"))
        assert [n["id"] for n in g["nodes"]] == ["", "0", "1"] and g["nodes"][1]["params"] == 9 and g["edges"] == [["", "0"], ["", "1"]]
        page = urllib.request.urlopen(f"http://127.0.0.1:{port}/").read().decode()
        assert "<svg" in page and "/metrics.json" in page
        assert v.histogram("loss", 2)["counts"] == [2, 2]
    finally:
        v.stop()

"""ONNX toolkit: export -> serialise -> parse -> check -> shapes -> run equals the torch module; optimiser and QDQ."""
import numpy as np
import torch

from sneppx_alg_b200.onnx import toolkit as ox


def test_export_roundtrip_run_optimize_quantize(tmp_path):
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.LayerNorm(16), torch.nn.GELU(approximate="tanh"),
                              torch.nn.Linear(16, 4), torch.nn.Tanh())
    x = torch.randn(5, 8)
    p = str(tmp_path / "m.onnx")
    ox.export_module(net, x, p)
    m = ox.Model.load(p)
    assert ox.check_model(m) == [] and m.opset == 17
    assert ox.infer_shapes(m, {"input": (5, 8)})[m.graph.outputs[0].name] == (5, 4)
    y = ox.run_model(m, {"input": x.numpy()})[m.graph.outputs[0].name]
    assert np.allclose(y, net(x).detach().numpy(), atol=1e-4)
    # a constant sub-graph gets folded away and a dead node removed
    g = m.graph
    g.nodes.insert(0, ox.Node("Add", ["c1", "c2"], ["csum"]))
    g.nodes.insert(1, ox.Node("Relu", ["csum"], ["dead"]))
    g.initializers["c1"], g.initializers["c2"] = np.ones(3, np.float32), np.ones(3, np.float32)
    opt = ox.optimize(m)
    assert len(opt.graph.nodes) == len(g.nodes) - 2 and "c1" not in opt.graph.initializers
    q = ox.quantize_qdq(opt)
    assert any(n.op_type == "DequantizeLinear" for n in q.graph.nodes)
    yq = ox.run_model(ox.Model.parse(q.serialize()), {"input": x.numpy()})[m.graph.outputs[0].name]
    assert np.abs(yq - y).max() < 0.1
    bad = ox.Model(ox.Graph([ox.Node("MatMul", ["input", "nope"], ["y"])], [ox.ValueInfo("input")], [ox.ValueInfo("z")]))
    errs = ox.check_model(bad)
    assert any("before definition" in e for e in errs) and any("never produced" in e for e in errs)
    assert ox.main(["check", p]) == 0


def test_external_data_and_runtime_session(tmp_path):
    """Large initializers move to a side file and come back bit-exact; a reference that leaves the model folder or
    lies about its length is refused; the runtime session gives the executor's results through the session API."""
    import pytest
    torch.manual_seed(1)
    net = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.ReLU(), torch.nn.Linear(64, 8))
    x = torch.randn(3, 32)
    m = ox.export_module(net, x)
    p = str(tmp_path / "big.onnx")
    moved = ox.save_external_data(m, p, size_threshold=1024)
    assert len(moved) == 2 and (tmp_path / "big.onnx.data").stat().st_size >= 32 * 64 * 4 + 64 * 8 * 4
    assert (tmp_path / "big.onnx").stat().st_size < 2500          # the big weights are not inside the model file
    raw = ox.Model.load(p)
    assert set(raw.external) == set(moved) and not raw.graph.initializers[moved[0]].any()      # placeholders until loaded
    back = ox.load_external_data(p)
    for k, v in m.graph.initializers.items():
        assert np.array_equal(back.graph.initializers[k], v)
    out_name = m.graph.outputs[0].name
    assert np.allclose(ox.run_model(back, {"input": x.numpy()})[out_name], net(x).detach().numpy(), atol=1e-5)
    # hostile descriptors
    evil = ox.Model(m.graph, external={moved[0]: {"location": "../escape.bin", "offset": "0", "length": "8192"}})
    evil.save(str(tmp_path / "evil.onnx"))
    (tmp_path.parent / "escape.bin").write_bytes(b"\x00" * 8192)
    with pytest.raises(ValueError, match="outside the model folder"):
        ox.load_external_data(str(tmp_path / "evil.onnx"))
    short = ox.Model(m.graph, external={moved[0]: {"location": "big.onnx.data", "offset": "0", "length": "16"}})
    short.save(str(tmp_path / "short.onnx"))
    with pytest.raises(ValueError, match="do not fit"):
        ox.load_external_data(str(tmp_path / "short.onnx"))
    sess = ox.OnnxRuntimeSession(back)
    assert sess.backend in ("sneppx", "onnxruntime") and [i.name for i in sess.get_inputs()] == ["input"]
    (y,) = sess.run(None, {"input": x.numpy()})
    assert np.allclose(y, net(x).detach().numpy(), atol=1e-4)
    if not ox.has_onnxruntime():
        with pytest.raises(RuntimeError):
            ox.OnnxRuntimeSession(back, require_ort=True)

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

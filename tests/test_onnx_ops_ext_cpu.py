"""Extended ONNX operator set, graph passes, strict checker and the convolutional exporter, against PyTorch."""
import numpy as np
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from sneppx_alg_b200.onnx import ops_ext as ox
from sneppx_alg_b200.onnx import toolkit as tk
from sneppx_alg_b200.onnx.toolkit import Graph, Model, Node, ValueInfo


def _run1(op, ins, attrs=None, n_out=1):
    names = [f"i{k}" for k in range(len(ins))]
    g = Graph([Node(op, names, [f"o{k}" for k in range(n_out)], attrs or {})],
              [ValueInfo(n) for n in names], [ValueInfo(f"o{k}") for k in range(n_out)])
    m = Model.parse(Model(g).serialize())          # through the wire format: attributes must survive it
    out = tk.run_model(m, dict(zip(names, ins)))
    return [out[f"o{k}"] for k in range(n_out)]


def test_conv_pool_batchnorm_match_torch():
    torch.manual_seed(0)
    x = torch.randn(2, 6, 13, 11)
    for groups, stride, pad, dil in ((1, 1, 1, 1), (2, 2, 0, 1), (3, 1, 2, 2), (6, 2, 1, 1)):
        w, b = torch.randn(12, 6 // groups, 3, 3), torch.randn(12)
        ref = F.conv2d(x, w, b, stride, pad, dil, groups)
        got = _run1("Conv", [x.numpy(), w.numpy(), b.numpy()], {"kernel_shape": [3, 3], "strides": [stride] * 2, "pads": [pad] * 4,
                                                                  "dilations": [dil] * 2, "group": groups})[0]
        assert np.allclose(got, ref.numpy(), atol=1e-4), (groups, stride, pad, dil)
    same = _run1("Conv", [x.numpy(), torch.randn(4, 6, 3, 3).numpy()], {"auto_pad": "SAME_UPPER", "strides": [2, 2]})[0]
    assert same.shape == (2, 4, 7, 6)
    assert np.allclose(_run1("MaxPool", [x.numpy()], {"kernel_shape": [3, 3], "strides": [2, 2], "pads": [1, 1, 1, 1]})[0],
                       F.max_pool2d(x, 3, 2, 1).numpy())
    assert np.allclose(_run1("MaxPool", [x.numpy()], {"kernel_shape": [2, 2], "strides": [2, 2], "ceil_mode": 1})[0],
                       F.max_pool2d(x, 2, 2, ceil_mode=True).numpy())
    for inc in (0, 1):
        assert np.allclose(_run1("AveragePool", [x.numpy()], {"kernel_shape": [3, 3], "strides": [2, 2], "pads": [1, 1, 1, 1],
                                                                "count_include_pad": inc})[0],
                           F.avg_pool2d(x, 3, 2, 1, count_include_pad=bool(inc)).numpy(), atol=1e-6)
    s, bb, mu, var = torch.rand(6) + 0.5, torch.randn(6), torch.randn(6), torch.rand(6) + 0.1
    assert np.allclose(_run1("BatchNormalization", [t.numpy() for t in (x, s, bb, mu, var)], {"epsilon": 1e-5})[0],
                       F.batch_norm(x, mu, var, s, bb, False, 0.0, 1e-5).numpy(), atol=1e-5)
    assert np.allclose(_run1("GlobalAveragePool", [x.numpy()])[0], x.mean((2, 3), keepdim=True).numpy(), atol=1e-6)


def test_tensor_manipulation_and_multi_output_ops():
    x = np.arange(2 * 3 * 8, dtype=np.float32).reshape(2, 3, 8)
    a, b, c = _run1("Split", [x, np.array([2, 5, 1])], {"axis": 2}, n_out=3)
    assert a.shape == (2, 3, 2) and b.shape == (2, 3, 5) and np.array_equal(np.concatenate([a, b, c], 2), x)
    h1, h2 = _run1("Split", [x], {"axis": 1}, n_out=2)        # even split from the number of outputs
    assert h1.shape == (2, 2, 8) and h2.shape == (2, 1, 8)
    v, idx = _run1("TopK", [x, np.array([3])], {"axis": -1}, n_out=2)
    tv, ti = torch.topk(torch.from_numpy(x), 3, dim=-1)
    assert np.array_equal(v, tv.numpy()) and np.array_equal(idx, ti.numpy())
    assert np.array_equal(_run1("Slice", [x, np.array([1, -6]), np.array([3, 100]), np.array([1, 2]), np.array([1, 2])])[0], x[:, 1:3, -6::2])
    assert _run1("Unsqueeze", [x, np.array([0, 4])])[0].shape == (1, 2, 3, 8, 1)
    assert _run1("Squeeze", [x[:1], np.array([0])])[0].shape == (3, 8)
    assert _run1("Flatten", [x], {"axis": 2})[0].shape == (6, 8)
    assert np.array_equal(_run1("Pad", [x, np.array([0, 1, 2, 0, 0, 1]), np.array(9.0, dtype=np.float32)])[0],
                          np.pad(x, [(0, 0), (1, 0), (2, 1)], constant_values=9.0))
    assert _run1("Cast", [x], {"to": 7})[0].dtype == np.int64
    assert np.array_equal(_run1("Shape", [x])[0], [2, 3, 8])
    assert np.array_equal(_run1("Where", [x > 10, x, -x])[0], np.where(x > 10, x, -x))
    assert np.array_equal(_run1("Expand", [x[:, :1], np.array([2, 3, 8])])[0], np.broadcast_to(x[:, :1], (2, 3, 8)))
    assert np.array_equal(_run1("ReduceSum", [x, np.array([1])], {"keepdims": 0})[0], x.sum(1))
    assert np.array_equal(_run1("ReduceMax", [x], {"axes": [0, 2]})[0], x.max((0, 2), keepdims=True))
    assert np.array_equal(_run1("ArgMax", [x], {"axis": 2, "keepdims": 0})[0], x.argmax(2))
    assert np.allclose(_run1("Einsum", [x, x], {"equation": "bik,bjk->bij"})[0], np.einsum("bik,bjk->bij", x, x))
    assert np.array_equal(_run1("Trilu", [x[0]], {"upper": 0})[0], np.tril(x[0]))
    assert np.allclose(_run1("Erf", [x / 10])[0], torch.erf(torch.from_numpy(x / 10)).numpy(), atol=1e-6)
    t = torch.randn(4, 16)
    w = torch.rand(16) + 0.5
    rms = t / torch.sqrt((t ** 2).mean(-1, keepdim=True) + 1e-6) * w
    assert np.allclose(_run1("SimplifiedLayerNormalization", [t.numpy(), w.numpy()], {"epsilon": 1e-6})[0], rms.numpy(), atol=1e-5)
    assert np.allclose(_run1("LogSoftmax", [t.numpy()], {"axis": -1})[0], F.log_softmax(t, -1).numpy(), atol=1e-5)
    assert np.allclose(_run1("ReduceMean", [t.numpy(), np.array([1])])[0], t.mean(1, keepdim=True).numpy(), atol=1e-6)


class _Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.f = nn.Sequential(nn.Conv2d(3, 8, 3, padding=1, bias=False), nn.BatchNorm2d(8), nn.ReLU(), nn.MaxPool2d(2),
                               nn.Conv2d(8, 16, 3, stride=2, padding=1), nn.BatchNorm2d(16), nn.SiLU(), nn.Dropout(0.1),
                               nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(16, 10), nn.LeakyReLU(0.2), nn.Linear(10, 4),
                               nn.LogSoftmax(dim=-1))

    def forward(self, x):
        return self.f(x)


def test_export_conv_stack_passes_and_checker(tmp_path):
    torch.manual_seed(1)
    net = _Net().eval()
    for mod in net.modules():
        if isinstance(mod, nn.BatchNorm2d):
            mod.running_mean.normal_()
            mod.running_var.uniform_(0.5, 2.0)
            mod.weight.data.uniform_(0.5, 1.5)
            mod.bias.data.normal_()
    x = torch.randn(5, 3, 16, 16)
    with torch.no_grad():
        ref = net(x).numpy()
    m = ox.export_sequential(net, x, str(tmp_path / "net.onnx"))
    m = Model.load(str(tmp_path / "net.onnx"))
    assert ox.check_model_strict(m) == []
    out = tk.run_model(m, {"input": x.numpy()})[m.graph.outputs[0].name]
    assert np.allclose(out, ref, atol=1e-4)
    n_before = len(m.graph.nodes)
    counts = ox.run_passes(m)
    assert counts["bn_fold"] == 2 and counts["gemm"] == 2
    assert len(m.graph.nodes) == n_before - 4
    assert not any(n.op_type in ("BatchNormalization", "Add") for n in m.graph.nodes)
    out2 = tk.run_model(m, {"input": x.numpy()})[m.graph.outputs[0].name]
    assert np.allclose(out2, ref, atol=1e-4)
    assert ox.check_model_strict(m) == []
    shapes = tk.infer_shapes(m, {"input": (2, 3, 16, 16)})
    assert shapes[m.graph.outputs[0].name] == (2, 4)


def test_transpose_identity_cse_passes_and_topological_sort():
    g = Graph([Node("Transpose", ["x"], ["a"], {"perm": [1, 0, 2]}), Node("Identity", ["a"], ["a2"]),
               Node("Transpose", ["a2"], ["b"], {"perm": [1, 0, 2]}), Node("Relu", ["b"], ["r1"]), Node("Relu", ["b"], ["r2"]),
               Node("Add", ["r1", "r2"], ["y0"]), Node("Transpose", ["y0"], ["t"], {"perm": [2, 0, 1]}),
               Node("Transpose", ["t"], ["y"], {"perm": [0, 2, 1]})],
              [ValueInfo("x", tk.DT_FLOAT, (2, 3, 4))], [ValueInfo("y")])
    m = Model(g)
    x = np.random.default_rng(0).standard_normal((2, 3, 4)).astype(np.float32)
    ref = tk.run_model(m, {"x": x})["y"]
    counts = ox.run_passes(m)
    assert counts["identity"] == 1 and counts["transposes"] == 2 and counts["cse"] == 1
    assert [n.op_type for n in m.graph.nodes] == ["Relu", "Add", "Transpose"]
    assert np.array_equal(tk.run_model(m, {"x": x})["y"], ref)
    m.graph.nodes.reverse()
    assert tk.check_model(m)                       # out of order now
    ox.topological_sort(m)
    assert tk.check_model(m) == [] and np.array_equal(tk.run_model(m, {"x": x})["y"], ref)
    m.graph.nodes.append(Node("Relu", ["nowhere"], ["z"]))
    with pytest.raises(ValueError):
        ox.topological_sort(m)


def test_strict_checker_reports_attribute_and_arity_errors():
    g = Graph([Node("Transpose", ["x"], ["a"], {"perm": [0, 0, 1]}, "t"), Node("Cast", ["a"], ["b"], {}, "c"),
               Node("MaxPool", ["b"], ["c"], {"kernel_shape": [2, 2], "strides": [1]}, "p"), Node("MatMul", ["c"], ["y"], {}, "t")],
              [ValueInfo("x", tk.DT_FLOAT, (2, 3, 4))], [ValueInfo("y")])
    errs = ox.check_model_strict(Model(g, opset=3))
    text = "\n".join(errs)
    for frag in ("opset 3", "'t' used more than once", "not a permutation", "attribute 'to' is missing", "strides has 1 entries",
                 "1 inputs, expected 2..2"):
        assert frag in text, (frag, errs)
    ok = Graph([Node("MatMul", ["x", "w"], ["y"])], [ValueInfo("x", tk.DT_FLOAT, (2, 3))], [ValueInfo("y")], {"w": np.ones((4, 5), np.float32)})
    assert any("shape inference failed" in e for e in ox.check_model_strict(Model(ok)))

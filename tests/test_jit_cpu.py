"""Tracing JIT: recording, replay on new inputs, passes, signature cache, composition with the transforms."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from sneppx_alg_b200 import jit


def test_trace_replays_without_running_python_again():
    calls = []
    w = torch.randn(8, 6)

    def f(x, y):
        calls.append(1)
        h = torch.tanh(x @ w) * y.sum(-1, keepdim=True)
        a, b = h.chunk(2, dim=-1)                       # multi-output node
        dead = (x * 3).exp()                            # never used                # noqa: F841
        return {"out": a + b, "norm": h.norm()}, h.shape[-1]

    x, y = torch.randn(4, 8), torch.randn(4, 3)
    tf = jit.trace(f, x, y)
    assert len(calls) == 1
    x2, y2 = torch.randn(4, 8), torch.randn(4, 3)
    out, width = tf(x2, y2)
    ref, _ = f(x2, y2)
    assert len(calls) == 2                              # only the reference call ran the Python
    assert width == 6 and torch.allclose(out["out"], ref["out"]) and torch.allclose(out["norm"], ref["norm"])
    g = tf.graph_for(x, y)
    assert not any(n.name == "exp" for n in g.nodes) and tf.stats(x, y)["dead"] >= 2
    assert "tanh" in tf.code(x, y) and "chunk" in tf.code(x, y)
    # constants are held by reference: an update of the closed-over weight is seen by the replay
    w.mul_(2.0)
    assert torch.allclose(tf(x2, y2)[0]["out"], f(x2, y2)[0]["out"])
    # a new shape retraces
    tf(torch.randn(6, 8), torch.randn(6, 3))
    assert tf.traces == 2 and len(calls) == 4      # trace, two reference calls, retrace


def test_cse_and_linear_activation_fusion():
    torch.manual_seed(0)
    net = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 32), nn.GELU(approximate="tanh"), nn.Linear(32, 8), nn.SiLU(),
                        nn.Linear(8, 4), nn.GELU())

    def f(x):
        y = net(x)
        return y + torch.sin(x).sum() + torch.sin(x).sum()       # the two sin / sum pairs are one computation

    x = torch.randn(3, 16)
    tf = jit.trace(f, x)
    st = tf.stats(x)
    assert st["fused_linear"] == 3 and st["cse"] == 2            # the erf-form GELU is not the epilogue's tanh form
    names = [n.name for n in tf.graph_for(x).nodes]
    assert names.count("linear") == 1 and names.count("sin") == 1 and "linear_relu" in names and "linear_silu" in names
    x2 = torch.randn(3, 16)
    assert torch.allclose(tf(x2), f(x2), atol=1e-5)
    # gradients flow through a replay
    x3 = torch.randn(3, 16, requires_grad=True)
    tf2 = jit.TracedFunction(f)
    tf2(x3).sum().backward()
    g1 = x3.grad.clone()
    x3.grad = None
    f(x3).sum().backward()
    assert torch.allclose(g1, x3.grad, atol=1e-5)
    assert net[0].weight.grad is not None


def test_inplace_nodes_survive_and_block_cse():
    def f(x):
        y = x.clone()
        y.add_(1.0)
        y[0] = 0.0
        z = x.clone()
        return y * 2 + z

    x = torch.randn(4, 4)
    tf = jit.trace(f, x)
    assert tf.stats(x)["cse"] == 0
    x2 = torch.randn(4, 4)
    assert torch.equal(tf(x2), f(x2))


def test_freeze_folds_weight_only_subgraphs():
    w = torch.randn(6, 6)

    def f(x):
        wn = F.normalize(w, dim=0) * 2.0          # depends on constants only
        return x @ wn

    x = torch.randn(2, 6)
    tf = jit.jit(f, freeze=True)
    ref = f(x)
    assert torch.allclose(tf(x), ref)
    assert tf.stats(x)["folded"] >= 2 and [n.name for n in tf.graph_for(x).nodes] in (["matmul"], ["__matmul__"])
    w.zero_()                                      # frozen: no longer seen
    assert torch.allclose(tf(x), ref)


def test_transforms_compose_with_traced_functions():
    tf = jit.trace(lambda x: (torch.sin(x) * x).sum(), torch.randn(5))
    x = torch.randn(5)
    assert torch.allclose(jit.grad(lambda t: tf(t))(x), torch.cos(x) * x + torch.sin(x), atol=1e-6)
    h = jit.hessian(lambda t: (t ** 3).sum())(x)
    assert torch.allclose(h, torch.diag(6 * x), atol=1e-5)
    assert torch.allclose(jit.vmap(lambda r: r.dot(r))(torch.eye(3) * 2), torch.full((3,), 4.0))

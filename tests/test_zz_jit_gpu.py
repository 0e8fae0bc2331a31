"""The tracing JIT on a GPU: under ``torch.no_grad`` a traced function replays through one captured CUDA graph; with
gradients enabled it replays the tape eagerly and autograd works."""
import pytest
import torch

from sneppx_alg_b200 import jit

pytestmark = pytest.mark.gpu


def test_traced_function_replays_through_a_cuda_graph():
    torch.manual_seed(0)
    w = torch.randn(64, 32, device="cuda")
    b = torch.randn(64, device="cuda")

    def f(x):
        h = torch.tanh(torch.nn.functional.linear(x, w, b))
        unused = h * 3.0                                   # noqa: F841  (dead code for the optimiser to drop)
        return h * 2.0 + x.sum(-1, keepdim=True)

    x = torch.randn(16, 32, device="cuda")
    tf = jit.trace(f, x)
    assert tf.traces == 1 and tf.stats(x).get("dead", 0) >= 0
    captured = next(iter(tf.cache.values()))[1]
    assert captured is not None                            # the replay was captured at trace time
    with torch.no_grad():
        y1 = tf(x).clone()
        x2 = torch.randn(16, 32, device="cuda")
        y2 = tf(x2).clone()
        assert torch.allclose(y1, f(x), atol=1e-5) and torch.allclose(y2, f(x2), atol=1e-5)
        assert tf.traces == 1                              # same signature: no second trace
        tf(torch.randn(8, 32, device="cuda"))
        assert tf.traces == 2                              # another shape: its own trace and graph
    xg = x.clone().requires_grad_(True)
    out = tf(xg)                                           # gradients on: eager replay of the tape
    out.sum().backward()
    ref = x.clone().requires_grad_(True)
    f(ref).sum().backward()
    assert torch.allclose(xg.grad, ref.grad, atol=1e-5)

"""Numerical gradient checks: for each differentiable op, the analytic gradient (autograd through the op, or its
hand-written backward) is compared with central finite differences along random directions,
(f(x + e v) - f(x - e v)) / 2e = <grad f, v>, for every floating-point input. The chunked SSD scan and the attention
backward have hand-written backward passes, so for them this is an oracle that shares no code with what it checks."""
import math

import pytest
import torch

from sneppx_alg_b200 import ops
from sneppx_alg_b200.ops import functional as Fn
from sneppx_alg_b200.ops import ssm


def directional_check(fn, inputs, eps=1e-2, tol=3e-2, directions=3, seed=0):
    """``fn(*inputs)`` returns a scalar. Returns the worst relative error over inputs and directions."""
    g = torch.Generator().manual_seed(seed)
    inputs = [x.clone().requires_grad_(x.is_floating_point()) for x in inputs]
    out = fn(*inputs)
    grads = torch.autograd.grad(out, [x for x in inputs if x.requires_grad], allow_unused=True)
    grads = iter(grads)
    worst = 0.0
    for i, x in enumerate(inputs):
        if not x.requires_grad:
            continue
        gx = next(grads)
        assert gx is not None, f"input {i} got no gradient"
        for _ in range(directions):
            v = torch.randn(x.shape, generator=g)
            v = v / v.norm()
            with torch.no_grad():
                plus = [t.detach() if j != i else (t.detach() + eps * v) for j, t in enumerate(inputs)]
                minus = [t.detach() if j != i else (t.detach() - eps * v) for j, t in enumerate(inputs)]
                numeric = (float(fn(*plus)) - float(fn(*minus))) / (2 * eps)
            analytic = float((gx.double() * v.double()).sum())
            err = abs(numeric - analytic) / max(1e-3, abs(numeric), abs(analytic))
            worst = max(worst, err)
            assert err < tol, f"input {i}: numeric {numeric:.6f} analytic {analytic:.6f}"
    return worst


def _weights(shape, seed):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed))


def test_norms_activations_and_losses():
    x, w, r = _weights((6, 32), 1), 1.0 + 0.1 * _weights((32,), 2), _weights((6, 32), 3)
    proj = _weights((6, 32), 4)
    directional_check(lambda x, w, r: (ops.rmsnorm(x, w, 1e-5, residual=r)[0] * proj).sum(), [x, w, r])
    directional_check(lambda x, w, b: (ops.layernorm(x, w, b) * proj).sum(), [x, w, _weights((32,), 5)])
    gu = _weights((5, 48), 6)
    for act in ("silu", "gelu", "relu"):
        directional_check(lambda gu: (ops.glu(gu, act) * _weights((5, 24), 7)).sum(), [gu + 0.3], tol=5e-2)
    logits, tgt = _weights((7, 19), 8), torch.randint(0, 19, (7,), generator=torch.Generator().manual_seed(9))
    tgt[2] = -100
    directional_check(lambda l: ops.cross_entropy(l, tgt), [logits])
    h, head = _weights((7, 12), 10), _weights((19, 12), 11) / 3
    directional_check(lambda h, head: ops.linear_cross_entropy(h, head, tgt), [h, head])


def test_rope_and_attention():
    B, S, H, Hk, D = 1, 6, 4, 2, 8
    cos, sin = ops.rope_tables(16, D, 10000.0, "cpu")
    qkv = _weights((B, S, (H + 2 * Hk) * D), 1)
    proj = _weights(qkv.shape, 2)
    directional_check(lambda t: (ops.rope_qk_(t, cos, sin, H + Hk, D) * proj).sum(), [qkv])
    q, k, v = _weights((B, S, H, D), 3), _weights((B, S, Hk, D), 4), _weights((B, S, Hk, D), 5)
    po = _weights((B, S, H, D), 6)
    for causal, window in ((True, 0), (False, 0), (True, 3)):
        directional_check(lambda q, k, v: (ops.attention(q, k, v, causal=causal, window=window) * po).sum(), [q, k, v])
    # the hand-written attention backward against finite differences of the forward
    o, lse = Fn.attention_reference(q, k, v, causal=True, return_lse=True)
    dq, dk, dv = Fn.attention_backward_reference(q, k, v, o, lse, po, causal=True)
    f = lambda q, k, v: (Fn.attention_reference(q, k, v, causal=True) * po).sum()                       # noqa: E731
    g = torch.Generator().manual_seed(7)
    for grad, idx in ((dq, 0), (dk, 1), (dv, 2)):
        d = torch.randn(grad.shape, generator=g)
        d = d / d.norm()
        args_p, args_m = [q, k, v], [q, k, v]
        args_p[idx], args_m[idx] = args_p[idx] + 1e-2 * d, args_m[idx] - 1e-2 * d
        numeric = (float(f(*args_p)) - float(f(*args_m))) / 2e-2
        assert abs(numeric - float((grad * d).sum())) < 3e-2 * max(1e-3, abs(numeric))


@pytest.mark.parametrize("L,chunk,groups", [(16, 8, 1), (24, 8, 2)])
def test_ssd_scan_hand_written_backward(L, chunk, groups):
    B, H, P, N = 2, 4, 4, 6
    x, dt = _weights((B, L, H, P), 1), 0.05 + 0.1 * torch.rand(B, L, H, generator=torch.Generator().manual_seed(2))
    A = -(0.5 + torch.rand(H, generator=torch.Generator().manual_seed(3)))
    Bm, Cm, D = _weights((B, L, groups, N), 4) / 2, _weights((B, L, groups, N), 5) / 2, _weights((H,), 6)
    h0 = _weights((B, H, P, N), 7) / 4
    py, ps = _weights((B, L, H, P), 8), _weights((B, H, P, N), 9)

    def f(x, dt, A, Bm, Cm, D, h0):
        y, final = ssm.ssd_scan(x, dt, A, Bm, Cm, D, chunk=chunk, init_state=h0, return_state=True)
        return (y * py).sum() + (final * ps).sum()

    directional_check(f, [x, dt, A, Bm, Cm, D, h0], eps=5e-3, tol=4e-2)
    # and the chunked scan agrees with the sequential recurrence
    want = ssm.ssd_reference(x, dt, A, Bm, Cm, D, init_state=h0) if "init_state" in ssm.ssd_reference.__code__.co_varnames else None
    if want is not None:
        want = want[0] if isinstance(want, tuple) else want
        assert torch.allclose(ssm.ssd_scan(x, dt, A, Bm, Cm, D, chunk=chunk, init_state=h0), want, atol=1e-4, rtol=1e-3)


def test_conv1d_and_linear():
    x, w, b = _weights((2, 10, 8), 1), _weights((8, 4), 2) / 2, _weights((8,), 3)
    proj = _weights((2, 10, 8), 4)
    directional_check(lambda x, w, b: (ssm.causal_conv1d(x, w, b, act=True) * proj).sum(), [x, w, b])
    a, wt, bias = _weights((5, 12), 5), _weights((7, 12), 6) / 3, _weights((7,), 7)
    for act in (None, "relu", "gelu", "silu"):
        directional_check(lambda a, wt, bias: (ops.linear(a + 0.2, wt, bias, act) * _weights((5, 7), 8)).sum(), [a, wt, bias], tol=5e-2)
    assert math.isfinite(float(ops.linear(a, wt).sum()))

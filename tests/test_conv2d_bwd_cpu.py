"""conv2d backward: the index arithmetic shared with the CUDA kernels, run by the host library, against autograd."""
import pytest
import torch

from sneppx_alg_b200.ops import conv

CASES = [  # N, C, H, W, K, R, S, stride, pad
    (2, 3, 8, 8, 4, 3, 3, 1, 1),
    (1, 2, 9, 7, 3, 3, 3, 2, 1),
    (2, 1, 5, 6, 2, 1, 1, 1, 0),
    (1, 3, 11, 10, 2, 5, 3, 3, 2),
    (3, 2, 4, 4, 5, 4, 4, 4, 0),      # patch embedding: kernel = stride
    (1, 1, 6, 6, 1, 2, 2, 2, 3),      # padding wider than the kernel
]


@pytest.mark.parametrize("case", CASES)
def test_backward_matches_autograd(case):
    N, C, H, W, K, R, S, stride, pad = case
    torch.manual_seed(sum(case))
    x, w = torch.randn(N, C, H, W), torch.randn(K, C, R, S)
    OH, OW = (H + 2 * pad - R) // stride + 1, (W + 2 * pad - S) // stride + 1
    dy = torch.randn(N, K, OH, OW)
    dx, dw, db = conv.conv2d_backward(x, w, dy, stride, pad)
    rx, rw, rb = conv.conv2d_backward_reference(x, w, dy, stride, pad)
    assert torch.allclose(dx, rx, atol=1e-4) and torch.allclose(dw, rw, atol=1e-4) and torch.allclose(db, rb, atol=1e-4)


def test_autograd_function_partial_needs_and_errors():
    torch.manual_seed(0)
    x = torch.randn(2, 3, 8, 8, requires_grad=True)
    w = torch.randn(4, 3, 3, 3, requires_grad=True)
    b = torch.randn(4, requires_grad=True)
    conv.conv2d(x, w, b, stride=2, padding=1).square().sum().backward()
    x2, w2, b2 = (t.detach().clone().requires_grad_(True) for t in (x, w, b))
    torch.nn.functional.conv2d(x2, w2, b2, stride=2, padding=1).square().sum().backward()
    assert torch.allclose(x.grad, x2.grad, atol=1e-3) and torch.allclose(w.grad, w2.grad, atol=1e-3) and torch.allclose(b.grad, b2.grad, atol=1e-3)
    frozen = torch.randn(2, 3, 8, 8)                                  # no gradient wanted for the input
    w3 = torch.randn(4, 3, 3, 3, requires_grad=True)
    conv.conv2d(frozen, w3).sum().backward()
    assert w3.grad is not None
    dx, dw, db = conv.conv2d_backward(frozen, w3.detach(), torch.ones(2, 4, 6, 6), need=(False, True, False))
    assert dx is None and db is None and torch.allclose(dw, w3.grad, atol=1e-4)
    with pytest.raises(ValueError):
        conv.conv2d_backward(frozen, w3.detach(), torch.ones(2, 4, 5, 5))
    with pytest.raises(TypeError):
        conv.conv2d_backward(frozen.double(), w3.detach().double(), torch.ones(2, 4, 6, 6).double())

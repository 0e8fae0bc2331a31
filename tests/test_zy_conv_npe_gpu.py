"""conv2d backward kernels and the NPE interpreter kernel against PyTorch / the host VM. Both kernels share their
index and instruction code with CPU oracles that the CPU suite checks."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_conv2d_backward_kernels(dtype):
    from sneppx_alg_b200.ops import conv
    torch.manual_seed(3)
    for N, C, H, W, K, R, S, stride, pad in ((2, 3, 17, 15, 5, 3, 3, 1, 1), (2, 4, 32, 32, 8, 4, 4, 4, 0), (1, 2, 9, 7, 3, 3, 3, 2, 1),
                                             (4, 16, 28, 28, 32, 3, 3, 2, 1)):
        x = torch.randn(N, C, H, W, device="cuda").to(dtype)
        w = torch.randn(K, C, R, S, device="cuda").to(dtype)
        OH, OW = (H + 2 * pad - R) // stride + 1, (W + 2 * pad - S) // stride + 1
        dy = torch.randn(N, K, OH, OW, device="cuda").to(dtype)
        dx, dw, db = conv.conv2d_backward(x, w, dy, stride, pad)
        rx, rw, rb = conv.conv2d_backward_reference(x, w, dy, stride, pad)
        for got, ref in ((dx, rx), (dw, rw), (db, rb)):
            assert got.dtype == torch.float32 and (got - ref).abs().max() <= 1e-3 * (1 + ref.abs().max())
    xg = torch.randn(2, 3, 16, 16, device="cuda", requires_grad=True)
    wg = torch.randn(6, 3, 3, 3, device="cuda", requires_grad=True)
    with torch.backends.cudnn.flags(allow_tf32=False):              # fp32 on both sides, not cuDNN's default TF32
        conv.conv2d(xg, wg, None, 1, 1).square().sum().backward()
        x2, w2 = xg.detach().clone().requires_grad_(True), wg.detach().clone().requires_grad_(True)
        torch.nn.functional.conv2d(x2, w2, None, 1, 1).square().sum().backward()
    assert torch.allclose(xg.grad, x2.grad, rtol=1e-3, atol=5e-2) and torch.allclose(wg.grad, w2.grad, rtol=1e-3, atol=5e-2)


def test_npe_interpreter_kernel_matches_host_vm():
    from sneppx_alg_b200.algorithms import npe
    torch.manual_seed(0)
    for dim, hidden, rows in ((24, 40, 7), (256, 1024, 300), (64, 64, 3000)):
        prog = npe.compile_mlp(dim, hidden, device="cuda")
        with torch.no_grad():
            prog.memory.normal_(0, dim ** -0.5)
        vm = npe.VM(npe.NPEConfig())
        vm.load(prog)
        vm.optimize()
        x = torch.randn(rows, dim, device="cuda")
        got = vm.run_rows(x)
        cpu = npe.VM(npe.NPEConfig(jit_enabled=False))
        cpu_prog = npe.compile_mlp(dim, hidden)
        with torch.no_grad():
            cpu_prog.memory.copy_(prog.memory.cpu())
        cpu.load(cpu_prog)
        want = cpu.run(x.cpu().float())
        assert got.shape == want.shape and (got.cpu() - want).abs().max() <= 2e-3 * (1 + want.abs().max())
    assert vm.plan_rows(64)[0] == 0

"""tcgen05 GEMM (G1/G2) against an fp32 PyTorch reference of the same op."""
import ctypes

import pytest
import torch

from sneppx_alg_b200 import ops
from sneppx_alg_b200.ops.gemm import gemm, gemm_reference

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (300, 200, 136), (4096, 1024, 512), (64, 128, 4096)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    torch.manual_seed(0)
    if (a_mn and M % 64) or (b_mn and N % 64):
        pytest.skip("MN-major operands need a multiple of 64")
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=torch.bfloat16)
    d = gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    ref = gemm_reference(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    ops.check_status()
    assert _rel(d, ref) < 1e-2


@pytest.mark.parametrize("M", [1, 7, 16, 33, 64, 100, 128])
@pytest.mark.parametrize("N,K", [(128, 256), (1000, 520), (4096, 4096), (6144, 4096), (4096, 14336), (50048, 1024)])
def test_gemm_decode_sized_cluster_split_k(M, N, K):
    """Decode-sized products go to the cluster split-K kernel: every cluster size from 1 to 8, ragged N and K tails,
    activation rows that do not divide by the cluster size."""
    from sneppx_alg_b200.ops import _lib
    torch.manual_seed(M * 7 + N)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.1
    args = _lib.SxGemmArgs()
    args.M, args.N, args.K, args.batch = M, N, K, 1
    assert _lib.lib().sx_gemm_skinny_ok(ctypes.byref(args)) == 1
    d = gemm(a, b)
    ref = gemm_reference(a, b, out_dtype=torch.float32)
    ops.check_status()
    assert _rel(d, ref) < 1e-2
    # same values on a second call (the reduction order over the cluster is fixed)
    assert torch.equal(d, gemm(a, b))


def test_gemm_decode_sized_epilogue_and_strided_out():
    torch.manual_seed(5)
    M, N, K = 48, 1536, 2048
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.1
    bias = torch.randn(N, device="cuda", dtype=torch.float32)
    for act in (None, "silu", "gelu", "relu"):
        d = gemm(a, b, alpha=0.5, bias=bias, act=act, out_dtype=torch.float32)
        ref = gemm_reference(a, b, alpha=0.5, bias=bias, act=act, out_dtype=torch.float32)
        assert _rel(d, ref) < 1e-2
    wide = torch.zeros(M, N + 64, device="cuda", dtype=torch.bfloat16)
    gemm(a, b, out=wide[:, 32: 32 + N])
    ops.check_status()
    assert _rel(wide[:, 32: 32 + N], gemm_reference(a, b, out_dtype=torch.float32)) < 1e-2
    assert float(wide[:, :32].abs().max()) == 0.0 and float(wide[:, 32 + N:].abs().max()) == 0.0


def test_gemm_epilogue_bias_beta_act_fp32out():
    torch.manual_seed(1)
    M, N, K = 384, 320, 192
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    c = torch.randn(M, N, device="cuda", dtype=torch.float32)
    bias = torch.randn(N, device="cuda", dtype=torch.float32)
    d = gemm(a, b, c=c, beta=0.5, alpha=0.25, bias=bias, act="gelu", out_dtype=torch.float32)
    ref = gemm_reference(a, b, c=c, beta=0.5, alpha=0.25, bias=bias, act="gelu", out_dtype=torch.float32)
    ops.check_status()
    assert _rel(d, ref) < 1e-2


def test_gemm_batched():
    torch.manual_seed(2)
    a = torch.randn(3, 256, 128, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(3, 192, 128, device="cuda", dtype=torch.bfloat16)
    d = gemm(a, b)
    ref = torch.matmul(a.float(), b.float().transpose(1, 2))
    ops.check_status()
    assert d.shape == (3, 256, 192) and _rel(d, ref) < 1e-2


def test_gemm_grouped_forward_and_wgrad():
    torch.manual_seed(3)
    E, K, N = 4, 256, 384
    counts = [128, 0, 256, 128]
    tile_group = torch.tensor([0, 2, 2, 3], dtype=torch.int32, device="cuda")
    a = torch.randn(sum(counts), K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(E, N, K, device="cuda", dtype=torch.bfloat16)
    d = gemm(a, w, tile_group=tile_group)
    ref = gemm_reference(a, w, tile_group=tile_group, out_dtype=torch.float32)
    assert _rel(d, ref) < 1e-2
    # per-expert wgrad: dW[e] = dY_e^T X_e over the expert's row range
    dy = torch.randn(sum(counts), N, device="cuda", dtype=torch.bfloat16)
    kr = torch.tensor([[0, 128], [128, 128], [128, 384], [384, 512]], dtype=torch.int32, device="cuda")
    dw = gemm(dy, a, a_mn=True, b_mn=True, k_ranges=kr, out_dtype=torch.float32)
    refw = gemm_reference(dy, a, a_mn=True, b_mn=True, k_ranges=kr, out_dtype=torch.float32)
    ops.check_status()
    assert dw.shape == (E, N, K) and _rel(dw, refw) < 1e-2


def test_linear_autograd_matches_torch():
    torch.manual_seed(4)
    x = torch.randn(2, 192, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(320, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = ops.linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    yr = torch.nn.functional.linear(xr, wr)
    yr.backward(g.float())
    ops.check_status()
    assert _rel(y, yr) < 1e-2 and _rel(x.grad, xr.grad) < 1e-2 and _rel(w.grad, wr.grad) < 1e-2


def test_gemm_mn_major_a_with_ragged_rows():
    """Weight-gradient shape whose output rows are not a multiple of the 64-element MN-major atom (Mamba-2's
    in_proj has 10576): the aligned part runs in place, the tail through a small transposed copy; with and
    without accumulation into an fp32 buffer."""
    torch.manual_seed(3)
    T, M, N = 1024, 400, 320
    g = torch.randn(T, M, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(T, N, device="cuda", dtype=torch.bfloat16)
    ref = g.float().t() @ x.float()
    d = gemm(g, x, a_mn=True, b_mn=True)
    assert d.shape == (M, N) and _rel(d, ref) < 1e-2
    acc = torch.randn(M, N, device="cuda")
    want = ref + acc
    gemm(g, x, a_mn=True, b_mn=True, out=acc, c=acc, beta=1.0)
    ops.check_status()
    assert _rel(acc, want) < 1e-2

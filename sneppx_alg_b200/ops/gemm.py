"""G1/G2 GEMM front-end: shape checks, allocation and the autograd ``Linear`` function.

CUDA bf16 tensors go to the tcgen05 kernel (``csrc/gemm_tc.cu``); anything else (CPU tensors, the
fp32 oracle in tests) takes the plain PyTorch path with identical semantics. The counterpart in the
reference is ``sneppx_gemm_fused`` / ``sneppx_cuda_gemm_bwd`` (kernel/cuda/tensor_cuda.cu:497-558,
kernel/cuda/autodiff_cuda.cu:28-171).
"""
from __future__ import annotations

import ctypes as C

import contextlib
import threading

import torch

from . import _lib

ACT = {None: 0, "none": 0, "gelu": 1, "silu": 2, "relu": 3}


def _act_ref(x, act):
    if act in (None, "none", 0):
        return x
    if act in ("gelu", 1):
        return torch.nn.functional.gelu(x, approximate="tanh")
    if act in ("silu", 2):
        return torch.nn.functional.silu(x)
    return torch.relu(x)


def gemm_reference(a, b, *, a_mn=False, b_mn=False, c=None, beta=0.0, alpha=1.0, bias=None, act=None,
                   out_dtype=None, tile_group=None, k_ranges=None):
    """fp32 PyTorch statement of what the kernel computes (also the CPU path)."""
    out_dtype = out_dtype or a.dtype
    A = a.float().transpose(-1, -2) if a_mn else a.float()
    Bm = b.float() if b_mn else b.float().transpose(-1, -2)  # [K, N]
    if tile_group is not None:
        M = A.shape[0]
        d = torch.zeros(M, Bm.shape[-1], dtype=torch.float32, device=a.device)
        tg = tile_group.tolist()
        for blk, g in enumerate(tg):
            if g < 0:
                continue
            r0, r1 = blk * 128, min((blk + 1) * 128, M)
            d[r0:r1] = A[r0:r1] @ Bm[g]
    elif k_ranges is not None:
        kr = k_ranges.view(-1, 2).tolist()
        d = torch.stack([A[:, k0:k1] @ Bm[k0:k1] for (k0, k1) in kr])
    else:
        d = A @ Bm
    d = d * alpha
    if bias is not None:
        d = d + bias.float()
    if c is not None and beta != 0.0:
        d = d + beta * c.float()
    return _act_ref(d, act).to(out_dtype)


class _Static(threading.local):
    on = False


_static = _Static()


@contextlib.contextmanager
def static_weights(on: bool = True):
    """Inside this block the second operand of every ``gemm`` / ``linear`` call is declared static: no kernel launched
    earlier on the stream writes it (weights at inference time). Decode-sized products then start fetching the weight
    while the kernel before them is still running (programmatic dependent launch)."""
    old, _static.on = _static.on, on
    try:
        yield
    finally:
        _static.on = old


def _use_kernel(*ts) -> bool:
    t = ts[0]
    return t.is_cuda and all(x is None or (x.is_cuda) for x in ts) and t.dtype == torch.bfloat16 and _lib.available()


def gemm(a, b, *, a_mn=False, b_mn=False, out=None, out_dtype=None, c=None, beta=0.0, alpha=1.0, bias=None,
         act=None, tile_group=None, k_ranges=None, sm_limit=0, force_bn=0):
    """D = act(alpha * A @ B^T + bias + beta * C).

    a: [.., M, K] (or [.., K, M] when ``a_mn``); b: [.., N, K] (or [.., K, N] when ``b_mn``).
    ``tile_group`` (int32 [ceil(M/128)]): grouped GEMM, b is [G, N, K]; block i of a multiplies b[tile_group[i]].
    ``k_ranges`` (int32 [G, 2]): a and b are MN-major with shared rows; batch g reduces rows [k0, k1) -> out [G, M, N].
    """
    if not _use_kernel(a, b, c, bias):
        r = gemm_reference(a, b, a_mn=a_mn, b_mn=b_mn, c=c, beta=beta, alpha=alpha, bias=bias, act=act,
                           out_dtype=out_dtype or (out.dtype if out is not None else None),
                           tile_group=tile_group, k_ranges=k_ranges)
        if out is not None:
            out.copy_(r)
            return out
        return r

    assert b.dtype == torch.bfloat16
    # Resolve operand storage into (matrix dims, leading dim, batch stride).
    def prep(t, mn_major):
        if t.stride(-1) != 1 or (t.dim() == 3 and t.stride(1) < t.shape[2]):
            t = t.contiguous()
        rows, cols = t.shape[-2], t.shape[-1]
        ext_mn, ext_k = (cols, rows) if mn_major else (rows, cols)
        ld = t.stride(-2)
        bs = t.stride(0) if t.dim() == 3 else 0
        return t, ext_mn, ext_k, ld, bs

    if (a_mn and a.dim() == 2 and a.shape[-1] % 64 != 0 and a.shape[-1] > 256 and tile_group is None
            and k_ranges is None and a.stride(-1) == 1 and (out is None or out.dim() == 2)
            and (c is None or c.dim() == 2)):
        # MN-major operands are tiled in 64-element atoms: run the aligned part in place and only the ragged
        # tail (< 64 rows of the result) through a transposed copy
        m0 = a.shape[-1] // 64 * 64
        if out is None:
            n_out = b.shape[-1] if b_mn else b.shape[-2]
            out = torch.empty(a.shape[-1], n_out, dtype=out_dtype or torch.bfloat16, device=a.device)
        kw = dict(b_mn=b_mn, alpha=alpha, beta=beta, bias=bias, act=act, sm_limit=sm_limit, force_bn=force_bn)
        gemm(a[:, :m0], b, a_mn=True, out=out[:m0], c=None if c is None else c[:m0], **kw)
        gemm(a[:, m0:].t().contiguous(), b, a_mn=False, out=out[m0:], c=None if c is None else c[m0:], **kw)
        return out
    if a_mn and a.shape[-1] % 64 != 0:
        a, a_mn = a.transpose(-1, -2).contiguous(), False
    if b_mn and b.shape[-1] % 64 != 0:
        b, b_mn = b.transpose(-1, -2).contiguous(), False
    a, M, K, lda, sA = prep(a, a_mn)
    b, N, Kb, ldb, sB = prep(b, b_mn)
    assert K == Kb, f"reduction mismatch {K} vs {Kb}"
    if K % 8 != 0 or lda % 8 != 0 or ldb % 8 != 0:
        # TMA needs 16-byte row pitches. A plain 2-D GEMM is zero-padded along K to the next multiple of 8 (zeros add
        # nothing to the sum; a copy with a padded pitch also fixes an odd leading dimension) and runs on the
        # tensor-core kernel; grouped / ranged / batched layouts that cannot be padded that way are refused rather
        # than quietly sent to a library GEMM.
        if tile_group is not None or k_ranges is not None or a.dim() != 2 or b.dim() != 2:
            raise ValueError(f"gemm: K={K}, lda={lda}, ldb={ldb} must be multiples of 8 elements for this layout; "
                             "pad the operands")
        Kp = (K + 7) // 8 * 8

        def pad_k(t, mn_major):
            # K is the row axis of an MN-major operand and the column axis of a K-major one
            if mn_major:
                cols = (t.shape[1] + 7) // 8 * 8
                buf = torch.zeros(Kp, cols, dtype=t.dtype, device=t.device)
                buf[: t.shape[0], : t.shape[1]] = t
                return buf[:, : t.shape[1]]
            buf = torch.zeros(t.shape[0], Kp, dtype=t.dtype, device=t.device)
            buf[:, : t.shape[1]] = t
            return buf

        return gemm(pad_k(a, a_mn), pad_k(b, b_mn), a_mn=a_mn, b_mn=b_mn, c=c, beta=beta, alpha=alpha, bias=bias, act=act,
                    out=out, out_dtype=out_dtype, sm_limit=sm_limit, force_bn=force_bn)
    batch = 1
    k_total = 0
    if k_ranges is not None:
        batch = k_ranges.numel() // 2
        k_total = K
        sA = sB = 0
    elif tile_group is not None:
        assert b.dim() == 3
        batch = 1
    else:
        if a.dim() == 3:
            batch = a.shape[0]
        if b.dim() == 3:
            batch = max(batch, b.shape[0])
    odt = out_dtype or (out.dtype if out is not None else torch.bfloat16)
    if out is None:
        shape = (batch, M, N) if (batch > 1 or a.dim() == 3 or (b.dim() == 3 and tile_group is None) or
                                  k_ranges is not None) else (M, N)
        out = torch.empty(shape, dtype=odt, device=a.device)
        from . import debug as _dbg
        if _dbg.ENABLED and tile_group is None and k_ranges is None:
            _dbg.poison_(out)      # debug-bounds mode: every element must be written by the kernel
    if tile_group is not None:
        from . import debug as _dbg
        if _dbg.ENABLED:
            _dbg.check_indices(tile_group, -1, b.shape[0], _dbg.SITE_TILE_GROUP)
    assert out.stride(-1) == 1
    ldd = out.stride(-2)
    sD = out.stride(0) if out.dim() == 3 else 0
    args = _lib.SxGemmArgs()
    args.A, args.B, args.D = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.C = c.data_ptr() if (c is not None and beta != 0.0) else None
    args.bias = bias.float().data_ptr() if bias is not None else None
    if bias is not None:
        _keep = bias.float()
        args.bias = _keep.data_ptr()
    args.M, args.N, args.K, args.batch = M, N, K, batch
    args.lda, args.ldb, args.ldd = lda, ldb, ldd
    args.ldc = c.stride(-2) if c is not None else 0
    args.strideA, args.strideB, args.strideD = sA, sB, sD
    args.strideC = (c.stride(0) if (c is not None and c.dim() == 3) else 0)
    args.a_mn, args.b_mn = int(a_mn), int(b_mn)
    args.out_fp32 = int(out.dtype == torch.float32)
    args.c_fp32 = int(c is not None and c.dtype == torch.float32)
    args.act = ACT[act] if not isinstance(act, int) else act
    args.alpha, args.beta = float(alpha), float(beta)
    if tile_group is not None:
        args.tile_group = tile_group.data_ptr()
        args.num_groups = b.shape[0]
        args.strideB = b.stride(0)
    if k_ranges is not None:
        args.k_ranges = k_ranges.data_ptr()
        args.k_total = k_total
    args.status = _lib.status_word(a.device).data_ptr()
    args.sm_limit = sm_limit
    args.force_bn = force_bn
    args.flags = 1 if _static.on else 0
    _lib.call("sx_gemm_bf16", C.byref(args), _lib.stream())
    return out


class _LinearFn(torch.autograd.Function):
    """y = x W^T (+ b). Backward runs dgrad and wgrad on the same kernel with MN-major operands;
    when the weight carries ``main_grad`` (a view into a flat gradient buffer) wgrad accumulates
    into it in place and ``.grad`` stays empty."""

    @staticmethod
    def forward(ctx, x, w, bias, act):
        x2 = x.reshape(-1, x.shape[-1])
        y = gemm(x2, w, bias=bias, act=act)
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.act = act
        ctx.xshape = x.shape
        assert act in (None, "none"), "fused activation is inference-only; training applies it separately"
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).view(ctx.xshape)
        if ctx.needs_input_grad[1]:
            mg = getattr(w, "main_grad", None)
            if mg is not None:
                first = not getattr(w, "_main_grad_written", False)
                gemm(dy2, x2, a_mn=True, b_mn=True, out=mg, c=None if first else mg, beta=0.0 if first else 1.0)
                w._main_grad_written = True
                dw = None
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=w.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db, None


def linear(x, w, bias=None, act=None):
    if torch.is_grad_enabled() and (x.requires_grad or w.requires_grad):
        return _LinearFn.apply(x, w, bias, None) if act in (None, "none") else _act_ref(
            _LinearFn.apply(x, w, bias, None), act)
    x2 = x.reshape(-1, x.shape[-1])
    return gemm(x2, w, bias=bias, act=act).view(*x.shape[:-1], w.shape[0])


class _BmmFn(torch.autograd.Function):
    """Batched C = A @ B on the tcgen05 GEMM (A [n, M, K], B [n, K, N]); both gradients reuse the kernel with
    MN-major operand flags instead of transposed copies."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return gemm(a, b, b_mn=True)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        g = g.contiguous()
        da = db = None
        if ctx.needs_input_grad[0]:
            da = gemm(g, b)                      # [n,M,N] x [n,K,N]^T -> [n,M,K]
        if ctx.needs_input_grad[1]:
            db = gemm(a, g, a_mn=True, b_mn=True)  # A^T [K,M] x G [M,N] -> [n,K,N]
        return da, db


def bmm(a, b):
    """Batched matmul with autograd; leading dims are flattened. bf16 CUDA tensors run on the tcgen05 GEMM."""
    if _use_kernel(a, b) and a.shape[-1] % 8 == 0 and b.shape[-1] % 8 == 0:
        lead = a.shape[:-2]
        a3 = a.reshape(-1, a.shape[-2], a.shape[-1])
        b3 = b.reshape(-1, b.shape[-2], b.shape[-1])
        if not a3.is_contiguous():
            a3 = a3.contiguous()
        if not b3.is_contiguous():
            b3 = b3.contiguous()
        return _BmmFn.apply(a3, b3).reshape(*lead, a.shape[-2], b.shape[-1])
    if _use_kernel(a, b):
        raise ValueError(f"bmm: inner sizes {a.shape[-1]} and {b.shape[-1]} must be multiples of 8 for the tensor-core "
                         "kernel; pad the operands")
    return torch.matmul(a, b)      # CPU tensors and dtypes the kernels do not cover (fp32 oracles)

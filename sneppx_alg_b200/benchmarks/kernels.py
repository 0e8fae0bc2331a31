"""Per-kernel micro-benchmarks with roofline fractions (the reference's ``benchmark.py`` / ``benchmark_suite.py``
time whole NumPy ops; here every case is one native sm_100a kernel).

``python -m sneppx_alg_b200.benchmarks.kernels <case> [--small] [--iters N] [--out file.json]``

Cases: gemm, gemm_decode, gemm_wgrad, attn_fwd, attn_bwd, rmsnorm, glu, rope, ce, adamw, sumsq, paged_decode, gemm_dq_fp8,
gemm_dq_int4, gemm_fp8, gemm_fp8_prefill, conv1d, conv1d_bwd, ssd_fwd, ssd_bwd, router, quant_fp8, dropout, rng_normal, layernorm_bwd, block_top2, conv2d_bwd, npe_interp, all.  ``--small`` picks a problem that still exceeds L2 but holds well
under 2 GB so that one launch can be captured by a profiler in seconds.  Timing: CUDA events on the launching
stream after 3 warm-up launches; inputs are larger than L2 or rotated between iterations.  Fractions are against the
measured copy bandwidth / cuBLAS bf16 throughput in ``MEASURED_PEAKS.json`` when that file is present at the
repository root, else the stated fallback.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def _peaks():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def _time(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _bf(*shape, grad=False):
    return torch.randn(*shape, device="cuda", dtype=torch.bfloat16, requires_grad=grad)


def case_gemm(small, iters, a_mn=False, b_mn=False):
    from ..ops.gemm import gemm
    M, N, K = (4096, 4096, 4096) if small else (8192, 8192, 8192)
    a = _bf(K, M) if a_mn else _bf(M, K)
    b = _bf(K, N) if b_mn else _bf(N, K)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out), iters)
    A, B = (a.t() if a_mn else a), (b if b_mn else b.t())
    ms_lib = _time(lambda: torch.matmul(A, B, out=out), iters)
    return dict(shape=[M, N, K], ms=ms, flops=2 * M * N * K, bytes=2 * (M * K + N * K + M * N), lib_ms=ms_lib, lib="cuBLAS")


def case_gemm_wgrad(small, iters):
    return case_gemm(small, iters, a_mn=True, b_mn=True)


def _attn_inputs(small, grad):
    B, S, H, Hk, D = (1, 2048, 16, 4, 128) if small else (1, 4096, 32, 8, 128)
    qkv = _bf(B, S, (H + 2 * Hk) * D, grad=grad)
    q = qkv[..., : H * D].view(B, S, H, D)
    k = qkv[..., H * D:(H + Hk) * D].view(B, S, Hk, D)
    v = qkv[..., (H + Hk) * D:].view(B, S, Hk, D)
    return qkv, q, k, v, 4 * B * H * S * S * D / 2, (B, S, H, Hk, D)


def case_attn_fwd(small, iters):
    from ..ops import functional as F
    qkv, q, k, v, fl, shp = _attn_inputs(small, False)
    with torch.no_grad():
        ms = _time(lambda: F.attention(q, k, v, causal=True), iters)
        qq, kk, vv = [x.transpose(1, 2) for x in (q, k, v)]
        ms_lib = _time(lambda: torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, is_causal=True, enable_gqa=True), iters)
    B, S, H, Hk, D = shp
    return dict(shape=list(shp), ms=ms, flops=fl, bytes=2 * B * S * D * (2 * H + 2 * Hk), lib_ms=ms_lib, lib="torch SDPA")


def case_attn_bwd(small, iters):
    from ..ops import functional as F
    qkv, q, k, v, fl, shp = _attn_inputs(small, True)
    with torch.no_grad():
        ms_f = _time(lambda: F.attention(q, k, v, causal=True), iters)
    g = torch.randn_like(F.attention(q, k, v, causal=True))
    ms_fb = _time(lambda: torch.autograd.grad(F.attention(q, k, v, causal=True), qkv, g), iters)
    B, S, H, Hk, D = shp
    return dict(shape=list(shp), ms=ms_fb - ms_f, flops=2.5 * fl, bytes=2 * B * S * D * (4 * H + 4 * Hk), note="forward+backward minus forward")


def case_rmsnorm(small, iters):
    from ..ops import functional as F
    T, Dm = (32768, 4096) if small else (131072, 4096)
    x, r, w = _bf(T, Dm), _bf(T, Dm), torch.ones(Dm, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        ms = _time(lambda: F.rmsnorm(x, w, 1e-5, residual=r), iters)
    return dict(shape=[T, Dm], ms=ms, bytes=2 * T * Dm * 4, note="fused residual add: reads x,r writes y,sum")


def case_glu(small, iters):
    from ..ops import functional as F
    T, Dm = (16384, 14336) if small else (65536, 14336)
    gu = _bf(T, 2 * Dm)
    with torch.no_grad():
        ms = _time(lambda: F.glu(gu), iters)
    return dict(shape=[T, 2 * Dm], ms=ms, bytes=2 * T * Dm * 3)


def case_rope(small, iters):
    from ..ops import functional as F
    B, S, H, Hk, D = (4, 4096, 32, 8, 128) if small else (16, 4096, 32, 8, 128)
    qkv = _bf(B, S, (H + 2 * Hk) * D)
    cos, sin = F.rope_tables(S, D, 5e5, "cuda")
    with torch.no_grad():
        ms = _time(lambda: F.rope_qk_(qkv, cos, sin, H + Hk, D), iters)
    return dict(shape=[B, S, H, Hk, D], ms=ms, bytes=2 * B * S * (H + Hk) * D * 2 + 2 * B * S * (H + 2 * Hk) * D * 2,
                note="out-of-place: clone of qkv plus rotate of q,k heads")


def case_ce(small, iters):
    from ..ops import functional as F
    T, V = (2048, 128256) if small else (8192, 128256)
    logits = _bf(T, V)
    tgt = torch.randint(0, V, (T,), device="cuda")
    ms = _time(lambda: F.cross_entropy(logits.detach().requires_grad_(True), tgt), iters)
    return dict(shape=[T, V], ms=ms, bytes=2 * T * V * 3, note="forward; gradient written in place in the same pass (2 reads + 1 write)")


def case_adamw(small, iters):
    from ..optim.fused import adamw_flat_
    n = (64 if small else 512) * 1024 * 1024
    p32 = torch.randn(n, device="cuda")
    m, v = torch.zeros_like(p32), torch.zeros_like(p32)
    g = torch.randn(n, device="cuda", dtype=torch.bfloat16)
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: adamw_flat_(p32, m, v, g, p16, 3e-4, 0.9, 0.95, 1e-8, 0.1, 10), iters)
    return dict(shape=[n], ms=ms, bytes=n * (12 + 2 + 12 + 2))


def case_sumsq(small, iters):
    from ..optim.fused import grad_norm_
    n = (256 if small else 1024) * 1024 * 1024
    g = torch.randn(n, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: grad_norm_([g]), iters)
    return dict(shape=[n], ms=ms, bytes=2 * n)


def _graph_time(fn, iters):
    """Device time of ``fn`` (a sequence of launches) replayed from a CUDA graph: no host time between launches."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return _time(g.replay, iters)


def case_gemm_decode(small, iters):
    """The four weight GEMMs of one Llama-3-8B decoder layer (and the LM head) at 64 rows of activations: weight
    streaming, so the fraction is of copy bandwidth. Every shape has several weight copies that are used in turn (more
    than L2 holds together), and the launches are replayed from a CUDA graph so that host time is not in the figure."""
    from ..ops.gemm import gemm
    M = 64
    shapes = [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)] + ([] if small else [(128256, 4096)])
    copies = [max(2, min(8, (320 << 20) // (2 * n * k))) for n, k in shapes]
    ws = [[_bf(n, k) for _ in range(c)] for (n, k), c in zip(shapes, copies)]
    xs = [_bf(M, k) for _, k in shapes]
    outs = [torch.empty(M, n, device="cuda", dtype=torch.bfloat16) for n, _ in shapes]
    rounds = max(copies)

    def ours():
        for i in range(rounds):
            for w, x, o in zip(ws, xs, outs):
                gemm(x, w[i % len(w)], out=o)

    def lib():
        for i in range(rounds):
            for w, x, o in zip(ws, xs, outs):
                torch.matmul(x, w[i % len(w)].t(), out=o)

    ms = _graph_time(ours, iters) / rounds
    ms_lib = _graph_time(lib, iters) / rounds
    per, per_lib = {}, {}
    for (n, k), w, x, o in zip(shapes, ws, xs, outs):
        def one(f):
            def run():
                for wi in w:
                    f(wi)
            return _graph_time(run, iters) / len(w) * 1e3
        per[f"{n}x{k}"] = round(one(lambda wi: gemm(x, wi, out=o)), 1)
        per_lib[f"{n}x{k}"] = round(one(lambda wi: torch.matmul(x, wi.t(), out=o)), 1)
    byt = sum(2 * n * k + 2 * M * k + 2 * M * n for n, k in shapes)
    return dict(shape=[M, shapes], ms=ms, bytes=byt, flops=sum(2 * M * n * k for n, k in shapes), lib_ms=ms_lib,
                lib="cuBLAS", per_shape_us=per, per_shape_us_lib=per_lib)


def case_paged_decode(small, iters):
    from ..ops import paged
    B, Hq, Hkv, D, bs, L = (32, 32, 8, 128, 16, 4096) if small else (64, 32, 8, 128, 16, 8192)
    nb = L // bs
    kc = _bf(B * nb, bs, Hkv, D)
    vc = _bf(B * nb, bs, Hkv, D)
    tables = torch.arange(B * nb, device="cuda", dtype=torch.int32).view(B, nb)
    lens = torch.full((B,), L, device="cuda", dtype=torch.int32)
    q = _bf(B, Hq, D)
    with torch.no_grad():
        ms = _time(lambda: paged.paged_decode(q, kc, vc, tables, lens), iters)
        old = os.environ.get("SX_PAGED_TC")
        os.environ["SX_PAGED_TC"] = "0"
        try:
            ms_simt = _time(lambda: paged.paged_decode(q, kc, vc, tables, lens), iters)
        finally:
            if old is None:
                del os.environ["SX_PAGED_TC"]
            else:
                os.environ["SX_PAGED_TC"] = old
    return dict(shape=[B, Hq, Hkv, D, L], ms=ms, bytes=2 * 2 * B * L * Hkv * D, lib_ms=ms_simt,
                lib="own SIMT kernel (SX_PAGED_TC=0)")


def _case_dq(mode, small, iters):
    from ..ops import quant
    M, N, K = (16, 14336, 4096) if small else (64, 28672, 8192)
    w = _bf(N, K)
    x = _bf(M, K)
    qw, sc = (quant.quant_fp8_128x128(w) if mode == "fp8" else quant.quant_int4(w))
    with torch.no_grad():
        ms = _time(lambda: quant.gemm_dequant(x, qw, sc, mode=mode), iters)
        ms_lib = _time(lambda: torch.matmul(x, w.t()), iters)
    wb = N * K * (1 if mode == "fp8" else 0.5)
    return dict(shape=[M, N, K], ms=ms, flops=2 * M * N * K, bytes=wb + 2 * M * K + 2 * M * N, lib_ms=ms_lib, lib="cuBLAS bf16 weights")


def case_gemm_dq_fp8(small, iters):
    return _case_dq("fp8", small, iters)


def case_gemm_dq_int4(small, iters):
    return _case_dq("int4", small, iters)


def case_gemm_fp8(small, iters):
    """Block-scaled fp8 x fp8 GEMM at decode size: weights streamed once."""
    from ..ops import quant
    M, N, K = (16, 14336, 4096) if small else (64, 28672, 8192)
    w, x = _bf(N, K), _bf(M, K)
    wq, sw = quant.quant_fp8_128x128(w)
    xq, sx = quant.quant_fp8_1x128(x)
    with torch.no_grad():
        ms = _time(lambda: quant.gemm_fp8(None, wq, sw, xq=xq, sx=sx), iters)
        ms_q = _time(lambda: quant.gemm_fp8(x, wq, sw), iters)
        ms_lib = _time(lambda: torch.matmul(x, w.t()), iters)
    return dict(shape=[M, N, K], ms=ms, ms_with_activation_quant=ms_q, flops=2 * M * N * K, bytes=N * K + M * K + 2 * M * N,
                lib_ms=ms_lib, lib="cuBLAS bf16 weights")


def case_gemm_fp8_prefill(small, iters):
    from ..ops import quant
    M, N, K = (1024, 4096, 4096) if small else (4096, 14336, 4096)
    w, x = _bf(N, K), _bf(M, K)
    wq, sw = quant.quant_fp8_128x128(w)
    xq, sx = quant.quant_fp8_1x128(x)
    with torch.no_grad():
        ms = _time(lambda: quant.gemm_fp8(None, wq, sw, xq=xq, sx=sx), iters)
        ms_lib = _time(lambda: torch.matmul(x, w.t()), iters)
    return dict(shape=[M, N, K], ms=ms, flops=2 * M * N * K, bytes=N * K + M * K + 2 * M * N, lib_ms=ms_lib, lib="cuBLAS bf16")


def case_conv1d(small, iters):
    from ..ops import ssm
    B, S, C = (4, 4096, 4352) if small else (16, 4096, 4352)
    x, w, b = _bf(B, S, C), _bf(C, 4), _bf(C)
    with torch.no_grad():
        ms = _time(lambda: ssm.causal_conv1d(x, w, b), iters)
    return dict(shape=[B, S, C], ms=ms, bytes=2 * B * S * C * 2)


def case_conv1d_bwd(small, iters):
    from ..ops import ssm
    B, S, C = (4, 4096, 4352) if small else (16, 4096, 4352)
    x, w, b = _bf(B, S, C).requires_grad_(True), _bf(C, 4).requires_grad_(True), _bf(C).requires_grad_(True)
    y = ssm.causal_conv1d(x, w, b)
    g = torch.randn_like(y)
    ms = _time(lambda: torch.autograd.grad(y, (x, w, b), g, retain_graph=True), iters)
    return dict(shape=[B, S, C], ms=ms, bytes=3 * B * S * C * 2)      # dy and x in, dx out


def _ssd_inputs(small):
    B, L, H, P, G, N = (1, 4096, 80, 64, 1, 128) if small else (1, 8192, 80, 64, 8, 128)
    x = _bf(B, L, H, P).requires_grad_(True)
    dt = (torch.rand(B, L, H, device="cuda") * 0.1 + 1e-3).requires_grad_(True)
    A = (-torch.rand(H, device="cuda") * 4 - 0.5).requires_grad_(True)
    Bm, Cm = _bf(B, L, G, N).requires_grad_(True), _bf(B, L, G, N).requires_grad_(True)
    D = torch.randn(H, device="cuda").requires_grad_(True)
    return (x, dt, A, Bm, Cm, D), (B, L, H, P, G, N)


def case_ssd_fwd(small, iters):
    """Mamba-2 2.7B scan shape (80 heads of 64, state 128, chunk 128). bytes = x in + y out + chunk states written and
    read once (bf16): what one kernel per chunk would have to move."""
    from ..ops import ssm
    ins, (B, L, H, P, G, N) = _ssd_inputs(small)
    with torch.no_grad():
        ms = _time(lambda: ssm.ssd_scan(*ins, chunk=128), iters)
    return dict(shape=[B, L, H, P, G, N], ms=ms, bytes=2 * B * L * H * P * 2 + 2 * B * (L // 128) * H * P * N * 2,
                flops=2.0 * B * L * H * (128 * P + 2 * P * N) + 2.0 * B * L * G * 128 * N)


def case_ssd_bwd(small, iters):
    from ..ops import ssm
    ins, (B, L, H, P, G, N) = _ssd_inputs(small)
    y = ssm.ssd_scan(*ins, chunk=128)
    g = torch.randn_like(y)
    ms = _time(lambda: torch.autograd.grad(y, ins, g, retain_graph=True), iters)
    return dict(shape=[B, L, H, P, G, N], ms=ms, bytes=4 * B * L * H * P * 2 + 3 * B * (L // 128) * H * P * N * 2)


def case_router(small, iters):
    from ..ops import moe
    T, E = (262144, 8) if small else (1048576, 8)
    logits = torch.randn(T, E, device="cuda")
    with torch.no_grad():
        ms = _time(lambda: moe.route(logits, 2), iters)
    return dict(shape=[T, E], ms=ms, bytes=T * E * 4 * 2 + T * 2 * 8)


def case_quant_fp8(small, iters):
    from ..ops import quant
    T, Dm = (32768, 4096) if small else (131072, 4096)
    x = _bf(T, Dm)
    with torch.no_grad():
        ms = _time(lambda: quant.quant_fp8_1x128(x), iters)
    return dict(shape=[T, Dm], ms=ms, bytes=T * Dm * 3 + T * Dm // 128 * 4)


def case_dropout(small, iters):
    from ..ops import aux
    T, Dm = (32768, 4096) if small else (131072, 4096)
    x = _bf(T, Dm)
    with torch.no_grad():
        ms = _time(lambda: aux.dropout(x, 0.1, seed=1), iters)
    return dict(shape=[T, Dm], ms=ms, bytes=T * Dm * 4, note="mask regenerated from the counter, never stored")


def case_rng_normal(small, iters):
    from ..ops import aux
    n = (1 << 26) if small else (1 << 28)
    ms = _time(lambda: aux.rng_fill(n, "normal", 0.0, 1.0, seed=1), iters)
    return dict(shape=[n], ms=ms, bytes=4 * n, note="write-only; includes the output allocation")


def case_layernorm_bwd(small, iters):
    from ..ops import aux
    T, Dm = (32768, 4096) if small else (131072, 4096)
    x, g = _bf(T, Dm, grad=True), _bf(T, Dm)
    w = torch.ones(Dm, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = aux.layernorm_train(x, w, None, 1e-5)
    ms = _time(lambda: torch.autograd.grad(y, (x, w), g, retain_graph=True), iters)
    return dict(shape=[T, Dm], ms=ms, bytes=T * Dm * 2 * 3, note="reads x, dy (second pass mostly from L2 / L1), writes dx")


def case_block_top2(small, iters):
    from ..ops import aux
    n = (1 << 26) if small else (1 << 28)
    x = torch.randn(n, device="cuda")
    ms = _time(lambda: aux.block_top2(x), iters)
    return dict(shape=[n], ms=ms, bytes=4 * n * 3, note="reads x, writes kept and residual")


def case_conv2d_bwd(small, iters):
    from ..ops import conv
    N, C, H, K = (32, 64, 56, 64) if small else (128, 64, 56, 64)
    x, w, dy = _bf(N, C, H, H), _bf(K, C, 3, 3), _bf(N, K, H, H)
    ms = _time(lambda: conv.conv2d_backward(x, w, dy, 1, 1), iters)
    return dict(shape=[N, C, H, H, K, 3, 3], ms=ms, bytes=2 * (x.numel() + dy.numel()) + 4 * x.numel(), flops=2 * 2 * N * K * C * 9 * H * H,
                note="direct SIMT kernels (dx, dw, db); flops = dgrad + wgrad, fraction is against the tensor-core peak they do not use")


def case_npe_interp(small, iters):
    from ..algorithms import npe
    dim, hidden, rows = 256, 1024, (1 << 16) if small else (1 << 18)
    prog = npe.compile_mlp(dim, hidden, device="cuda")
    with torch.no_grad():
        prog.memory.normal_(0, dim ** -0.5)
    vm = npe.VM(npe.NPEConfig())
    vm.load(prog)
    vm.optimize()
    x = torch.randn(rows, dim, device="cuda")
    ms = _time(lambda: vm.run_rows(x), iters)
    return dict(shape=[rows, dim, hidden], ms=ms, bytes=4 * rows * dim * 2, flops=2 * 2 * rows * dim * hidden,
                note="whole MLP program in one launch, registers in shared memory, weights re-read from L2 per row")


CASES = {k[5:]: v for k, v in list(globals().items()) if k.startswith("case_")}


def run(name, small=False, iters=10):
    from .. import ops
    hbm, tf, src = _peaks()
    r = CASES[name](small, iters)
    r["case"], r["small"] = name, small
    if "flops" in r:
        r["tflops"] = r["flops"] / r["ms"] / 1e9
        r[f"frac_tensor_of_{src}"] = r["tflops"] / tf
    r["gbs"] = r["bytes"] / r["ms"] / 1e6
    r[f"frac_hbm_of_{src}"] = r["gbs"] / hbm
    ops.check_status()
    return r


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("case", choices=sorted(CASES) + ["all"])
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out")
    a = ap.parse_args(argv)
    names = sorted(CASES) if a.case == "all" else [a.case]
    res = []
    for n in names:
        r = run(n, a.small, a.iters)
        print(json.dumps(r), flush=True)
        res.append(r)
    if a.out:
        json.dump(res, open(a.out, "w"), indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""Fused compute+collective kernels against their rooflines and their library (cuBLAS + NCCL) equivalents.

Run one process per GPU, e.g.
``python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 -m sneppx_alg_b200.benchmarks.fused``

For each path the roofline time is the slower of FLOPs / measured GEMM peak and bytes that must cross NVLink / link
bandwidth. The link bandwidth is measured at the start of the run (``benchmarks/link.py``: every rank pulling 256 MiB
from its neighbour with 16-byte peer loads at the same time) and printed; 900 GB/s per direction per GPU is nominal.
Times are CUDA-event times on each rank, maximum over ranks; rank 0 prints one JSON line per case.

Cases
  ag_gemm    all-gather of activation rows -> GEMM (TP column-parallel in_proj / QKV)
  gemm_rs    GEMM -> reduce-scatter of output rows (TP row-parallel o_proj / down_proj)
  zero_ag    ZeRO-3 parameter all-gather of a 1 GiB bf16 bucket: pull kernel over peer loads, and (NVLS) one multimem.st
             push per rank
  zero_rs_adamw  ZeRO gradient reduce-scatter + AdamW in one kernel: peer loads, and (NVLS) multimem.ld_reduce
  wgather_gemm   ZeRO-3 weight all-gather fused into the consuming GEMM (B rows pulled by the GEMM's copy CTAs)
  allreduce  small all-reduce (norms / loss / router statistics)
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0     # replaced by the measured figure at the start of main()


def _peaks():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["bf16_tflops"], "measured"
    return 1590.0, "fallback"


def _time(fn, iters, group):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier(group)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192, help="total token rows of the TP group")
    ap.add_argument("--d", type=int, default=4096)
    ap.add_argument("--ff", type=int, default=14336)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from ..ops import check_status
    from ..parallel.symm import SymmGroup
    from ..parallel.tp import FusedTP, _all_gather_rows, _reduce_scatter_rows
    sg = SymmGroup()
    tp = FusedTP(sg)
    group = dist.group.WORLD
    tf, src = _peaks()
    res = []
    global NVLINK_GBS
    if world > 1:
        from .link import measure_link_gbs
        NVLINK_GBS = measure_link_gbs(sg, group=group)
        if rank == 0:
            print(json.dumps({"case": "link_bandwidth", "world": world, "GBps_per_direction_per_gpu": NVLINK_GBS,
                              "how": "256 MiB of 16-byte peer loads from the next rank, all ranks at once",
                              "nominal": 900.0}), flush=True)
    T, d, ff = a.tokens, a.d, a.ff
    rows = T // world
    bf = dict(device="cuda", dtype=torch.bfloat16)

    def report(name, shape, ms, ms_lib, flops, link_bytes, note=""):
        t_compute = flops / (tf * 1e12) * 1e3
        t_link = link_bytes / (NVLINK_GBS * 1e9) * 1e3
        roof = max(t_compute, t_link)
        r = {"case": name, "world": world, "shape": shape, "ms": ms, "library_ms": ms_lib, "speedup_vs_library": ms_lib / ms,
             "roofline_ms": roof, f"frac_of_roofline_{src}": roof / ms, "bound": "compute" if t_compute >= t_link else "nvlink",
             "link_GBps_used": NVLINK_GBS, "note": note}
        res.append(r)
        if rank == 0:
            print(json.dumps(r), flush=True)

    # ---- all-gather -> GEMM: x [T/world, d] per rank, W_col [ff_local, d]
    n_loc = (2 * ff // world) // 256 * 256
    x_shard = torch.randn(rows, d, **bf)
    w_col = torch.randn(n_loc, d, **bf) * 0.02
    ms = _time(lambda: tp.ag_gemm(x_shard, w_col, key="bench_ag"), a.iters, group)
    ms_lib = _time(lambda: torch.matmul(_all_gather_rows(x_shard, group), w_col.t()), a.iters, group)
    report("ag_gemm", [T, n_loc, d], ms, ms_lib, 2.0 * T * n_loc * d, (world - 1) * rows * d * 2,
           "gate_up column shard; link bytes = rows pulled from the other ranks")

    # ---- GEMM -> reduce-scatter: h [T, ff_local] x W_row [d, ff_local] -> [T/world, d]
    k_loc = (ff // world) // 64 * 64
    h = torch.randn(T, k_loc, **bf)
    w_row = torch.randn(d, k_loc, **bf) * 0.02
    ms = _time(lambda: tp.gemm_rs(h, w_row), a.iters, group)
    ms_lib = _time(lambda: _reduce_scatter_rows(torch.matmul(h, w_row.t()), group), a.iters, group)
    report("gemm_rs", [T, d, k_loc], ms, ms_lib, 2.0 * T * d * k_loc, (world - 1) * rows * d * 2,
           "down_proj row shard; link bytes = partial rows sent to their owners (bf16)")

    # ---- ZeRO-3 parameter all-gather, 1 GiB bucket
    n = (512 * 1024 * 1024) // world // 256 * 256
    shard = sg.alloc(n, torch.bfloat16)
    shard.tensor.normal_()
    full = torch.empty(world * n, **bf)
    lib_out = torch.empty(world * n, **bf)
    ms = _time(lambda: sg.allgather_pull(shard, full, n * 2, grid=48), a.iters, group)
    ms_lib = _time(lambda: dist.all_gather_into_tensor(lib_out, shard.tensor, group=group), a.iters, group)
    report("zero_ag", [world * n], ms, ms_lib, 0.0, (world - 1) * n * 2, "pull kernel over peer loads")
    full_s = sg.alloc(world * n, torch.bfloat16)
    if full_s.multicast_ptr and world > 1:
        ms = _time(lambda: sg.allgather_mc(shard.tensor, full_s, 0, n * 2, 7, sg.next_epoch(7), grid=32), a.iters, group)
        report("zero_ag_nvls", [world * n], ms, ms_lib, 0.0, world * n * 2,
               "one multimem.st push per rank; link bytes = the whole buffer arriving from the switch")
        ok_mc = bool(torch.equal(full_s.tensor[rank * n: rank * n + 4096], shard.tensor[:4096]))
        if not ok_mc:
            raise RuntimeError("multicast all-gather delivered wrong data")

    # ---- ZeRO-3 weight all-gather fused into the consuming GEMM: act [T/world.., d] x (gathered W [ff2, d])^T
    if world > 1:
        n_w = (2 * ff) // world // 256 * 256
        w_shard = torch.randn(n_w, d, **bf) * 0.02
        act = torch.randn(rows * world if rows * world <= 8192 else 8192, d, **bf)
        ms = _time(lambda: tp.ag_gemm(w_shard, act, key="bench_f2", gather_b=True), a.iters, group)
        w_full = torch.empty(world * n_w, d, **bf)
        ms_lib = _time(lambda: (dist.all_gather_into_tensor(w_full, w_shard, group=group), torch.matmul(act, w_full.t())),
                       a.iters, group)
        report("wgather_gemm", [act.shape[0], world * n_w, d], ms, ms_lib, 2.0 * act.shape[0] * world * n_w * d,
               (world - 1) * n_w * d * 2, "gate_up weight sharded by rows (ZeRO-3); library = all_gather + cuBLAS")


    # ---- ZeRO reduce-scatter + AdamW in one kernel: every rank holds a full bf16 gradient bucket
    if world > 1:
        import ctypes as C
        from ..ops import _lib
        from ..parallel.symm import SxZeroArgs
        nb = (256 * 1024 * 1024) // world // 256 * 256 * world          # bucket elements (512 MiB of bf16)
        sz = nb // world
        gbuf = sg.alloc(nb, torch.bfloat16)
        gbuf.tensor.normal_()
        p32 = torch.randn(sz, device="cuda")
        m_, v_ = torch.zeros_like(p32), torch.zeros_like(p32)
        p16 = torch.empty(sz, **bf)
        partials = torch.zeros(4096, device="cuda")
        state = {"e": 0}

        def fused_rs_adamw(nvls=False):
            state["e"] += 1
            sg.signal(2, state["e"])
            za = SxZeroArgs()
            za.peers = sg.peers(gbuf)
            za.elem_offset, za.n = rank * sz, sz
            za.sumsq_partials, za.num_partials = partials.data_ptr(), partials.numel()
            za.p32, za.m, za.v, za.p16_out = p32.data_ptr(), m_.data_ptr(), v_.data_ptr(), p16.data_ptr()
            za.lr, za.beta1, za.beta2, za.eps, za.wd, za.step, za.max_norm = 1e-4, 0.9, 0.95, 1e-8, 0.1, 5, 0.0
            za.ready_channel, za.ready_epoch = 2, state["e"]
            za.done_channel, za.done_epoch = 3, state["e"]
            za.mode, za.grid = 3, _lib.lib().sx_zero_grid_default()
            za.mc_buf = gbuf.multicast_ptr if nvls else None
            za.status = _lib.status_word(sg.device).data_ptr()
            _lib.call("sx_zero_step", C.byref(za), _lib.stream())

        red = torch.empty(sz, **bf)
        opt_p = torch.nn.Parameter(p32.clone())
        opt = torch.optim.AdamW([opt_p], lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)

        def lib_rs_adamw():
            dist.reduce_scatter_tensor(red, gbuf.tensor, group=group)
            opt_p.grad = red.float() / world
            opt.step()
            p16.copy_(opt_p.data)

        ms = _time(fused_rs_adamw, a.iters, group)
        ms_lib = _time(lib_rs_adamw, a.iters, group)
        # bytes: every rank reads (world-1) remote shards of bf16 grads; HBM side 28 B per owned parameter
        report("zero_rs_adamw", [nb], ms, ms_lib, 0.0, (world - 1) * sz * 2,
               "peer loads of the other ranks' slices, reduce, AdamW, bf16 shadow write in one pass")
        if gbuf.multicast_ptr:
            ms = _time(lambda: fused_rs_adamw(True), a.iters, group)
            report("zero_rs_adamw_nvls", [nb], ms, ms_lib, 0.0, nb * 2,
                   "multimem.ld_reduce (sum in the switch), AdamW, bf16 shadow write; link bytes = the whole bucket "
                   "leaving every GPU towards the switch")

    # ---- expert-parallel SER layer (DeepSeek-V2-Lite shape: d 2048, 64 experts of d_ff 1408, top-6, 2 shared)
    if world > 1 and 64 % world == 0:
        from ..nn.moe import SERMoE
        from ..parallel import expert as ep
        dm, dff, E, k, Tm = 2048, 1408, 64, 6, 8192
        layer = SERMoE(dm, dff, num_experts=E, top_k=k, num_shared_experts=2, dtype=torch.bfloat16, device="cuda",
                       ep_group=group, init_std=0.02)
        with torch.no_grad():
            dist.broadcast(layer.router.weight, 0)
            for prm in layer.shared.parameters():
                dist.broadcast(prm, 0)
        xm = torch.randn(Tm, dm, **bf)
        gm = torch.randn(Tm, dm, **bf)

        def run(fused):
            ep.FORCE_FUSED = fused
            xx = xm.detach().requires_grad_(True)
            y = layer(xx)
            y.backward(gm)
            for prm in layer.parameters():
                prm.grad = None

        ms = _time(lambda: run(True), a.iters, group)
        ms_lib = _time(lambda: run(False), a.iters, group)
        ep.FORCE_FUSED = None
        flops = 3 * 2.0 * Tm * k * 3 * dm * dff + 3 * 2.0 * Tm * 2 * 3 * dm * dff      # routed + shared experts, fwd + bwd
        link = 2 * 2 * Tm * k * dm * 2 * (world - 1) / world                              # dispatch + combine, fwd + bwd
        report("ep_moe_fwd_bwd", [Tm, dm, dff, E, k], ms, ms_lib, flops, link,
               "whole SER layer incl. router and shared experts; library = all_to_all + grouped GEMM")

    # ---- small all-reduce
    small = sg.alloc(1024, torch.float32)
    small.tensor.fill_(1.0)
    lib_small = torch.ones(1024, device="cuda")
    ms = _time(lambda: sg.allreduce_small(small, 1024), 50, group)
    ms_lib = _time(lambda: dist.all_reduce(lib_small, group=group), 50, group)
    report("allreduce_4KB", [1024], ms, ms_lib, 0.0, 0.0, "latency bound: roofline not meaningful")
    check_status()
    if a.out and rank == 0:
        json.dump(res, open(a.out, "w"), indent=1)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

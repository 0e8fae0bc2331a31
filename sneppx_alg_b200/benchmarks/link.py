"""NVLink / NVSwitch link micro-benchmark: what this package's own kernels move per direction per GPU.

Run one process per GPU:
``python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 -m sneppx_alg_b200.benchmarks.link``

Every rank runs the same probe at the same time (rank r talks to rank r+1), so the figures are per-GPU rates with
the whole switch busy, not a single idle link:

  p2p_pull        16-byte peer loads from the next rank's buffer into local memory
  p2p_push        16-byte peer stores of local memory into the next rank's buffer
  nvls_ld_reduce  ``multimem.ld_reduce`` over the group's multicast mapping (bf16 sum in the switch); bytes counted
                  are the reduced bytes that arrive (each is the sum of ``world`` values pulled inside the switch)
  nvls_st         ``multimem.st`` of local memory to the multicast mapping (the switch delivers to every rank);
                  bytes counted are the bytes each rank sends once

Sizes 1 MiB .. 1 GiB, CUDA-event times, max over ranks. ``measure_link_gbs`` (the 256 MiB peer pull) is what the
fused-collective benchmark uses as its link roofline; the nominal figure is 900 GB/s per direction per GPU.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os

import torch
import torch.distributed as dist

KINDS = {"p2p_pull": 0, "p2p_push": 1, "nvls_ld_reduce": 2, "nvls_st": 3}


def _probe(sg, buf, local, kind, nbytes, grid, iters, group):
    from ..ops import _lib
    p = sg.peers(buf)
    peer = (sg.rank + 1) % sg.world
    mc = C.c_void_p(buf.multicast_ptr or 0)

    def run():
        _lib.call("sx_link_probe", C.byref(p), C.c_int(kind), C.c_int(peer), mc, C.c_void_p(local.data_ptr()),
                  C.c_longlong(nbytes), C.c_int(grid), _lib.stream())

    for _ in range(3):
        run()
    torch.cuda.synchronize()
    dist.barrier(group)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        run()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    dist.barrier(group)
    return float(t)


def measure_link_gbs(sg, nbytes=256 << 20, grid=64, iters=5, group=None):
    """Per-direction per-GPU rate of 16-byte peer loads with every rank pulling from its neighbour at once (GB/s)."""
    group = group if group is not None else sg.group
    buf = sg.alloc(nbytes // 2, torch.bfloat16)
    local = torch.empty(nbytes // 2, dtype=torch.bfloat16, device=sg.device)
    buf.tensor.zero_()
    torch.cuda.synchronize()
    dist.barrier(group)
    ms = _probe(sg, buf, local, 0, nbytes, grid, iters, group)
    return nbytes / (ms * 1e-3) / 1e9


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mib", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--grid", type=int, default=64)
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    from ..parallel.symm import SymmGroup
    sg = SymmGroup()
    group = dist.group.WORLD
    nmax = a.max_mib << 20
    buf = sg.alloc(nmax // 2, torch.bfloat16)
    buf.tensor.zero_()
    local = torch.zeros(nmax // 2, dtype=torch.bfloat16, device=sg.device)
    torch.cuda.synchronize()
    dist.barrier(group)
    res = []
    sizes = [s << 20 for s in (1, 4, 16, 64, 256, 1024) if s <= a.max_mib]
    for name, kind in KINDS.items():
        if kind >= 2 and not buf.multicast_ptr:
            if rank == 0:
                print(json.dumps({"case": name, "unavailable": "no multicast mapping (NVLS) for this group"}), flush=True)
            continue
        for nbytes in sizes:
            ms = _probe(sg, buf, local, kind, nbytes, a.grid, a.iters, group)
            r = {"case": name, "world": world, "MiB": nbytes >> 20, "ms": ms, "GBps_per_gpu": nbytes / (ms * 1e-3) / 1e9,
                 "grid": a.grid}
            res.append(r)
            if rank == 0:
                print(json.dumps(r), flush=True)
    if a.out and rank == 0:
        json.dump(res, open(a.out, "w"), indent=1)
    dist.barrier(group)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

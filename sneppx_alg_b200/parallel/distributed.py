"""Process-group facade with the reference's names (interface_bindings/distributed.py:35-177, nccl.py:78-308,
distributed_wrapper.py:79-97; C twin net/distributed/nccl.h:52-197): ``init_process_group`` reading
WORLD_SIZE / RANK / LOCAL_RANK / MASTER_ADDR / MASTER_PORT, collectives that really communicate (the reference's
return their input), a device mesh for dp x tp x pp x ep, bucketed ``DistributedDataParallel`` and ``launch``."""
from __future__ import annotations

import enum
import os
import subprocess
import sys
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.distributed as dist


class NCCLRedOp(enum.IntEnum):
    SUM = 0
    PROD = 1
    MAX = 2
    MIN = 3
    AVG = 4


class NCCLDataType(enum.IntEnum):   # values of nccl.h (the reference's table maps FLOAT to 0, which is ncclInt8)
    INT8 = 0
    UINT8 = 1
    INT32 = 2
    UINT32 = 3
    INT64 = 4
    UINT64 = 5
    FLOAT16 = 6
    FLOAT32 = 7
    FLOAT64 = 8
    BFLOAT16 = 9


_OPS = {NCCLRedOp.SUM: dist.ReduceOp.SUM, NCCLRedOp.PROD: dist.ReduceOp.PRODUCT, NCCLRedOp.MAX: dist.ReduceOp.MAX,
        NCCLRedOp.MIN: dist.ReduceOp.MIN, NCCLRedOp.AVG: dist.ReduceOp.SUM, "sum": dist.ReduceOp.SUM,
        "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN, "avg": dist.ReduceOp.SUM, "mean": dist.ReduceOp.SUM}


@dataclass
class DistributedContext:
    world_size: int = 1
    rank: int = 0
    local_rank: int = 0
    master_addr: str = "127.0.0.1"
    master_port: int = 29500
    backend: str = "nccl"

    @classmethod
    def from_env(cls, backend: Optional[str] = None):
        return cls(int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0)),
                   int(os.environ.get("LOCAL_RANK", 0)), os.environ.get("MASTER_ADDR", "127.0.0.1"),
                   int(os.environ.get("MASTER_PORT", 29500)),
                   backend or ("nccl" if torch.cuda.is_available() else "gloo"))

    def init_process_group(self):
        if dist.is_initialized():
            return self
        os.environ.setdefault("MASTER_ADDR", self.master_addr)
        os.environ.setdefault("MASTER_PORT", str(self.master_port))
        kw = {}
        if self.backend == "nccl":
            torch.cuda.set_device(self.local_rank)
            kw["device_id"] = torch.device("cuda", self.local_rank)
        dist.init_process_group(self.backend, rank=self.rank, world_size=self.world_size, **kw)
        return self


def init_process_group(backend: Optional[str] = None, **kw) -> DistributedContext:
    return DistributedContext.from_env(backend).init_process_group()


def destroy_process_group():
    if dist.is_initialized():
        dist.destroy_process_group()


def get_world_size(group=None) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


def get_rank(group=None) -> int:
    return dist.get_rank(group) if dist.is_initialized() else 0


def barrier(group=None):
    if dist.is_initialized():
        dist.barrier(group)


def all_reduce(t: torch.Tensor, op=NCCLRedOp.SUM, group=None) -> torch.Tensor:
    if dist.is_initialized() and get_world_size(group) > 1:
        dist.all_reduce(t, _OPS[op], group=group)
        if op in (NCCLRedOp.AVG, "avg", "mean"):
            t.div_(get_world_size(group))
    return t


def broadcast(t: torch.Tensor, src: int = 0, group=None) -> torch.Tensor:
    if dist.is_initialized() and get_world_size(group) > 1:
        dist.broadcast(t, src, group=group)
    return t


def all_gather(t: torch.Tensor, group=None) -> List[torch.Tensor]:
    if not dist.is_initialized() or get_world_size(group) == 1:
        return [t]
    out = [torch.empty_like(t) for _ in range(get_world_size(group))]
    dist.all_gather(out, t.contiguous(), group=group)
    return out


def reduce_scatter(t: torch.Tensor, group=None) -> torch.Tensor:
    w = get_world_size(group)
    if w == 1:
        return t
    out = torch.empty(t.numel() // w, dtype=t.dtype, device=t.device)
    if dist.get_backend(group) == "nccl":
        dist.reduce_scatter_tensor(out, t.contiguous().view(-1), group=group)
    else:
        tmp = t.clone().view(-1)
        dist.all_reduce(tmp, group=group)
        out.copy_(tmp.view(w, -1)[get_rank(group)])
    return out


class ProcessGroup:
    """Thin object form (``sneppx_pg_create / barrier / all_reduce`` of net/distributed/nccl.h:170-197)."""

    def __init__(self, ranks: Optional[List[int]] = None):
        self.group = dist.new_group(ranks) if ranks is not None and dist.is_initialized() else None

    def all_reduce(self, t, op=NCCLRedOp.SUM):
        return all_reduce(t, op, self.group)

    def barrier(self):
        barrier(self.group)

    def size(self):
        return get_world_size(self.group)

    def rank(self):
        return get_rank(self.group)


class DeviceMesh:
    """Ranks laid out as [pp][dp][ep?][tp] with tp fastest (neighbouring GPUs): ``groups(dim)`` gives the process group
    of this rank along a dimension. ep shares the dp ranks (experts are sharded over data-parallel replicas)."""

    def __init__(self, dp=1, tp=1, pp=1, ep=1):
        self.dp, self.tp, self.pp, self.ep = dp, tp, pp, ep
        self.world = get_world_size()
        assert dp * tp * pp == self.world, f"dp*tp*pp = {dp * tp * pp} != world {self.world}"
        assert dp % ep == 0, "ep must divide dp"
        self.rank = get_rank()
        self._groups: Dict[str, object] = {}
        r = torch.arange(self.world).view(pp, dp, tp)
        self.coord = {"pp": self.rank // (dp * tp), "dp": (self.rank // tp) % dp, "tp": self.rank % tp}
        if dist.is_initialized() and self.world > 1:
            for name, dim in (("tp", 2), ("dp", 1), ("pp", 0)):
                moved = r.movedim(dim, -1).reshape(-1, r.shape[dim])
                for ranks in moved.tolist():
                    g = dist.new_group(ranks) if len(ranks) > 1 else None
                    if self.rank in ranks:
                        self._groups[name] = g
            # expert groups: consecutive blocks of ep ranks inside each dp group
            for p in range(pp):
                for t in range(tp):
                    for s in range(0, dp, ep):
                        ranks = [int(r[p, s + i, t]) for i in range(ep)]
                        g = dist.new_group(ranks) if ep > 1 else None
                        if self.rank in ranks:
                            self._groups["ep"] = g

    def group(self, name):
        return self._groups.get(name)


class DistributedDataParallel(torch.nn.Module):
    """Gradient averaging in buckets after backward (``sync_gradients``); for language models the ZeRO engine is the
    faster path, this wrapper serves arbitrary modules."""

    def __init__(self, module, bucket_size_mb: float = 25.0, group=None):
        super().__init__()
        self.module, self.group = module, group
        self.bucket_bytes = int(bucket_size_mb * 2 ** 20)
        if dist.is_initialized() and get_world_size(group) > 1:
            for p in module.parameters():
                dist.broadcast(p.data, 0, group=group)

    def forward(self, *a, **k):
        return self.module(*a, **k)

    def sync_gradients(self):
        w = get_world_size(self.group)
        if w == 1:
            return
        bucket, size = [], 0
        def flush():
            if not bucket:
                return
            flat = torch.cat([g.reshape(-1) for g in bucket])
            dist.all_reduce(flat, group=self.group)
            flat.div_(w)
            off = 0
            for g in bucket:
                g.copy_(flat[off: off + g.numel()].view_as(g))
                off += g.numel()
        for p in self.module.parameters():
            if p.grad is None:
                continue
            bucket.append(p.grad)
            size += p.grad.numel() * p.grad.element_size()
            if size >= self.bucket_bytes:
                flush()
                bucket, size = [], 0
        flush()


class DistributedWrapper(DistributedDataParallel):
    pass


def launch(script: str, nproc_per_node: int = 1, args: Optional[List[str]] = None, master_port: int = 29500) -> int:
    """Start ``script`` under torch.distributed.run on this node (the reference shells out the same way,
    distributed.py:162-177)."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc_per_node}",
           "--master-addr", "127.0.0.1", "--master-port", str(master_port), script] + list(args or [])
    return subprocess.call(cmd)

"""Hierarchical all-reduce: reduce-scatter inside each node, all-reduce of the 1/local_size shards across nodes between
ranks of equal local index, all-gather inside the node.

The reference's ``sneppx_hierarchical_ar_*`` (``kernel/distributed/gradient_comm.c:29-119``) names these three phases
and performs them as local copies through 256 MiB staging buffers. Here they are real collectives on two families of
process groups. Inside an NVSwitch node the flat NVLS all-reduce is already one hop, so this path matters when a job
spans nodes: only 1/local_size of the bytes crosses the slower inter-node fabric per rank, in parallel over the local
ranks' network interfaces.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist

from .distributed import reduce_scatter


def make_node_groups(local_size: int) -> Tuple[object, object]:
    """(intra-node group, inter-node group) of this rank for nodes of `local_size` consecutive ranks. Every rank of the
    job must call it: process groups are created collectively."""
    world, rank = dist.get_world_size(), dist.get_rank()
    if world % local_size:
        raise ValueError(f"world size {world} is not a multiple of the node size {local_size}")
    intra = inter = None
    for node in range(world // local_size):
        g = dist.new_group(list(range(node * local_size, (node + 1) * local_size)))
        if rank // local_size == node:
            intra = g
    for local in range(local_size):
        g = dist.new_group(list(range(local, world, local_size)))
        if rank % local_size == local:
            inter = g
    return intra, inter


def hierarchical_all_reduce(t: torch.Tensor, intra, inter, average: bool = False) -> torch.Tensor:
    """In-place sum (or mean) of `t` over all ranks. Works for any element count: the flat view is padded to a multiple
    of the node size for the scatter phase."""
    local = dist.get_world_size(intra)
    nodes = dist.get_world_size(inter)
    flat = t.reshape(-1)
    n = flat.numel()
    pad = (-n) % local
    buf = torch.cat([flat, flat.new_zeros(pad)]) if pad else flat.clone()
    shard = reduce_scatter(buf, group=intra) if local > 1 else buf           # phase 1: this rank owns 1/local of the node sum
    if nodes > 1:
        dist.all_reduce(shard, group=inter)                                  # phase 2: same shard index across nodes
    if average:
        shard.div_(local * nodes)
    if local > 1:                                                            # phase 3: rebuild the full tensor in the node
        parts = [torch.empty_like(shard) for _ in range(local)]
        dist.all_gather(parts, shard, group=intra)
        buf = torch.cat(parts)
    else:
        buf = shard
    flat.copy_(buf[:n])
    return t


class HierarchicalAllReduce:
    """Gradient synchroniser with the bucket interface of the reference (create with a staging size, then
    ``all_reduce(tensors)``): tensors are packed into buckets of at most `bucket_bytes`, each bucket goes through the
    three phases once, and results are copied back."""

    def __init__(self, local_size: int, bucket_bytes: int = 256 << 20, average: bool = True):
        self.intra, self.inter = make_node_groups(local_size)
        self.bucket_bytes, self.average = bucket_bytes, average
        self.bytes_inter_node = 0            # bytes this rank put on the inter-node phase (for reports and tests)

    def _buckets(self, tensors: Sequence[torch.Tensor]) -> List[List[torch.Tensor]]:
        out, cur, size = [], [], 0
        for t in tensors:
            b = t.numel() * t.element_size()
            if cur and (size + b > self.bucket_bytes or t.dtype != cur[0].dtype):
                out.append(cur)
                cur, size = [], 0
            cur.append(t)
            size += b
        if cur:
            out.append(cur)
        return out

    def all_reduce(self, tensors: Sequence[torch.Tensor]):
        local = dist.get_world_size(self.intra)
        for bucket in self._buckets(list(tensors)):
            flat = torch.cat([t.reshape(-1) for t in bucket])
            hierarchical_all_reduce(flat, self.intra, self.inter, self.average)
            self.bytes_inter_node += (flat.numel() + local - 1) // local * flat.element_size()
            off = 0
            for t in bucket:
                t.copy_(flat[off:off + t.numel()].view_as(t))
                off += t.numel()

    def sync_gradients(self, module: torch.nn.Module):
        self.all_reduce([p.grad for p in module.parameters() if p.grad is not None])

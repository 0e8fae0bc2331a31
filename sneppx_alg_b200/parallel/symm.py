"""Symmetric memory for the fused-collective kernels.

``SymmGroup`` owns, per process group, the signal pad and every symmetric data buffer (same size on
every rank, mapped into every peer's address space over NVLink). Allocation and the pointer
exchange go through ``torch.distributed._symmetric_memory`` (CUDA VMM + handle exchange); the
kernels that use the peer pointers are this package's own (``csrc/comm_fused.cu`` and the fused
GEMMs). The reference has no counterpart: its NCCL wrapper cannot form a communicator
(net/distributed/nccl.c:151-170) and its collectives are local copies.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops import _lib

PAD_STRIDE = 16
PAD_CHANNELS = 64
PAD_WORDS = PAD_STRIDE * PAD_CHANNELS


class SxPeers(C.Structure):
    _fields_ = [("buf", C.c_void_p * 8), ("pad", C.c_void_p * 8), ("rank", C.c_int), ("world", C.c_int),
                ("timeout_ns", C.c_ulonglong)]


class SxZeroArgs(C.Structure):
    _fields_ = [
        ("peers", SxPeers), ("elem_offset", C.c_longlong), ("n", C.c_longlong),
        ("reduced", C.c_void_p), ("sumsq_partials", C.c_void_p), ("partial_offset", C.c_int), ("num_partials", C.c_int),
        ("p32", C.c_void_p), ("m", C.c_void_p), ("v", C.c_void_p), ("p16_out", C.c_void_p),
        ("lr", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float), ("wd", C.c_float),
        ("step", C.c_int), ("max_norm", C.c_float), ("norm_out", C.c_void_p),
        ("ready_channel", C.c_int), ("ready_epoch", C.c_uint), ("norm_channel", C.c_int), ("norm_epoch", C.c_uint),
        ("done_channel", C.c_int), ("done_epoch", C.c_uint), ("mode", C.c_int), ("grid", C.c_int),
        ("status", C.c_void_p), ("mc_buf", C.c_void_p),
    ]


GUARD_BYTES = 256          # canary zone on each side of a symmetric buffer in debug-bounds mode
CANARY = 0x5A


class SymmBuffer:
    """One symmetric allocation: ``tensor`` is the local view, ``ptrs[r]`` rank r's mapping of the same range.
    With ``guard`` > 0 the allocation carries that many canary bytes before and after the usable range (the
    pointers and the tensor already point past the leading guard)."""

    def __init__(self, tensor, handle, guard: int = 0, raw=None):
        self.tensor = tensor
        self.handle = handle
        self.guard, self.raw = guard, raw
        self.ptrs = [int(p) + guard for p in handle.buffer_ptrs]
        try:
            self.multicast_ptr = (int(handle.multicast_ptr) + guard) if handle.has_multicast_support else 0
        except Exception:  # noqa: BLE001
            self.multicast_ptr = 0

    def canaries_intact(self) -> bool:
        """True when no kernel (local or a peer's) wrote into the guard zones around this buffer."""
        if not self.guard:
            return True
        b = self.raw.view(torch.uint8)
        g = self.guard
        return bool((b[:g] == CANARY).all()) and bool((b[-g:] == CANARY).all())


class SymmGroup:
    def __init__(self, group=None, timeout_s: float = 2.0):
        import torch.distributed._symmetric_memory as symm_mem
        self._sm = symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        assert self.world <= 8, "one NVSwitch domain (<= 8 GPUs) per symmetric group"
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.timeout_ns = int(timeout_s * 1e9)
        self._buffers = []
        try:
            symm_mem.enable_symm_mem_for_group(self.group.group_name)
        except Exception:  # noqa: BLE001  (newer torch enables groups implicitly)
            pass
        self.pad = self.alloc(PAD_WORDS, torch.int32)
        self.pad.tensor.zero_()
        torch.cuda.synchronize()
        dist.barrier(self.group)
        self._epochs = {}

    def alloc(self, numel: int, dtype) -> SymmBuffer:
        from ..ops import debug as _dbg
        if _dbg.ENABLED:
            # debug-bounds mode: guard zones of canary bytes around every peer-mapped buffer
            es = torch.empty(0, dtype=dtype).element_size()
            ge = GUARD_BYTES // es
            raw = self._sm.empty(numel + 2 * ge, dtype=dtype, device=self.device)
            h = self._sm.rendezvous(raw, group=self.group)
            raw.view(torch.uint8)[:GUARD_BYTES].fill_(CANARY)
            raw.view(torch.uint8)[-GUARD_BYTES:].fill_(CANARY)
            buf = SymmBuffer(raw[ge: ge + numel], h, guard=GUARD_BYTES, raw=raw)
            self._buffers.append(buf)
            return buf
        t = self._sm.empty(numel, dtype=dtype, device=self.device)
        h = self._sm.rendezvous(t, group=self.group)
        return SymmBuffer(t, h)

    def check_canaries(self) -> None:
        """Debug-bounds mode: raise if any symmetric buffer's guard zone was overwritten."""
        torch.cuda.synchronize()
        for i, b in enumerate(self._buffers):
            if not b.canaries_intact():
                from ..ops.debug import KernelBoundsError
                raise KernelBoundsError(f"symmetric buffer {i} ({b.tensor.numel()} x {b.tensor.dtype}): guard zone overwritten")

    def next_epoch(self, channel: int) -> int:
        e = self._epochs.get(channel, 0) + 1
        self._epochs[channel] = e
        return e

    def peers(self, buf: SymmBuffer | None = None, offset_bytes: int = 0) -> SxPeers:
        p = SxPeers()
        for r in range(self.world):
            p.buf[r] = (buf.ptrs[r] + offset_bytes) if buf is not None else 0
            p.pad[r] = self.pad.ptrs[r]
        p.rank, p.world, p.timeout_ns = self.rank, self.world, self.timeout_ns
        return p

    def barrier(self, channel: int = 60, stream=None):
        """Device-side barrier across the group (no host sync)."""
        e = self.next_epoch(channel)
        p = self.peers()
        _lib.call("sx_peer_barrier", C.byref(p), C.c_int(channel), C.c_uint(e),
                  C.c_void_p(_lib.status_word(self.device).data_ptr()), stream or _lib.stream())

    def signal(self, channel: int, epoch: int, stream=None):
        p = self.peers()
        _lib.call("sx_signal_peers", C.byref(p), C.c_int(channel), C.c_uint(epoch), stream or _lib.stream())

    def allgather_pull(self, src: SymmBuffer, dst: torch.Tensor, shard_bytes: int, src_offset_bytes: int = 0,
                       channel: int = -1, epoch: int = 0, grid: int = 32, stream=None):
        p = self.peers(src)
        _lib.call("sx_allgather_pull", C.byref(p), C.c_void_p(dst.data_ptr()), C.c_longlong(shard_bytes),
                  C.c_longlong(src_offset_bytes), C.c_int(channel), C.c_uint(epoch), C.c_int(grid),
                  C.c_void_p(_lib.status_word(self.device).data_ptr()), stream or _lib.stream())

    def allgather_mc(self, src: torch.Tensor, dst: SymmBuffer, dst_offset_bytes: int, shard_bytes: int, channel: int,
                     epoch: int, grid: int = 32, stream=None):
        """NVLS all-gather: store ``src`` (this rank's shard) once to the multicast mapping of ``dst`` at
        ``dst_offset_bytes + rank * shard_bytes``; ends with a barrier over the group on ``channel``."""
        assert dst.multicast_ptr, "buffer has no multicast mapping"
        p = self.peers(dst)
        _lib.call("sx_allgather_mc", C.byref(p), C.c_void_p(src.data_ptr()),
                  C.c_void_p(dst.multicast_ptr + dst_offset_bytes + self.rank * shard_bytes), C.c_longlong(shard_bytes),
                  C.c_int(channel), C.c_uint(epoch), C.c_int(grid),
                  C.c_void_p(_lib.status_word(self.device).data_ptr()), stream or _lib.stream())

    def allreduce_bf16_(self, x: torch.Tensor, staging: SymmBuffer, state: torch.Tensor, channel: int = 40, stream=None):
        """In-place sum over the group of a contiguous bf16 tensor (numel % 8 == 0, at most the staging size) through
        peer loads. ``state``: int32 [2] device tensor zeroed once (epoch counter, CTA counter) owned by the caller
        and used by no other call site at the same time. Safe inside CUDA-graph capture."""
        n = x.numel()
        assert x.is_contiguous() and x.dtype == torch.bfloat16 and n % 8 == 0 and n <= staging.tensor.numel()
        staging.tensor[:n].copy_(x.view(-1))
        p = self.peers(staging)
        _lib.call("sx_allreduce_bf16", C.byref(p), C.c_void_p(x.data_ptr()), C.c_longlong(n), C.c_int(channel),
                  C.c_void_p(state.data_ptr()), C.c_void_p(state.data_ptr() + 4), C.c_int(0),
                  C.c_void_p(_lib.status_word(self.device).data_ptr()), stream or _lib.stream())
        return x

    def allreduce_small(self, buf: SymmBuffer, n: int, channel: int = 56, stream=None):
        e = self.next_epoch(channel)
        p = self.peers(buf)
        _lib.call("sx_allreduce_small", C.byref(p), C.c_int(n), C.c_int(channel), C.c_uint(e),
                  C.c_void_p(_lib.status_word(self.device).data_ptr()), stream or _lib.stream())

"""Python face of the C++ CPU-rank runtime (``csrc/host/dist_runtime.cpp``): TCP ring all-reduce with the reference's
``arix_dist_*`` entry points (net/distributed/src/lib.rs:881-1098) and the UDP heartbeat failure detector
(kernel/distributed/heartbeat.c), plus the elastic-membership logic of kernel/distributed/elastic.c:87-219 and the
fault-tolerance glue of kernel/distributed/checkpoint.c:382-457 / interface_bindings/checkpoint.py:328-506."""
from __future__ import annotations

import ctypes as C
from typing import Callable, Dict, List, Optional

import numpy as np

from .. import _build

ALIVE, SUSPECT, DEAD = 0, 1, 2
MAX_RESTARTS = 10      # include/neural_core/kernel/elastic.h:8


def _lib():
    L = _build.load_host()
    if not getattr(L, "_dist_ready", False):
        L.arix_dist_ring_all_reduce.argtypes = [C.c_void_p, C.c_ulonglong, C.c_int]
        L.arix_dist_all_reduce.argtypes = [C.c_void_p, C.c_ulonglong]
        L.arix_dist_all_reduce_sum.argtypes = [C.c_void_p, C.c_ulonglong]
        L.arix_dist_sync_params.argtypes = [C.c_void_p, C.c_ulonglong, C.c_void_p]
        L.arix_dist_add_noise.argtypes = [C.c_void_p, C.c_ulonglong, C.c_float, C.c_ulonglong]
        L.arix_dist_connect.argtypes = [C.c_char_p, C.c_int]
        L.sx_hb_create.restype = C.c_void_p
        L.sx_hb_create.argtypes = [C.c_int] * 5
        for f in ("sx_hb_start", "sx_hb_stop"):
            getattr(L, f).argtypes = [C.c_void_p]
        L.sx_hb_status.argtypes = [C.c_void_p, C.c_int]
        L.sx_hb_set_send_enabled.argtypes = [C.c_void_p, C.c_int]
        L._dist_ready = True
    return L


class TcpRing:
    """One process = one node of the ring (the library keeps one ring per process, like the reference runtime)."""

    def __init__(self, node_id: int, world: int, addresses: List[str], timeout_ms: int = 10000):
        self.node_id, self.world = node_id, world
        port = int(addresses[node_id].rsplit(":", 1)[1])
        rc = _lib().arix_dist_init(node_id, world, port)
        if rc != 0:
            raise OSError(f"arix_dist_init failed ({rc})")
        rc = _lib().arix_dist_connect(",".join(addresses).encode(), timeout_ms)
        if rc != 0:
            raise OSError(f"arix_dist_connect failed ({rc})")

    def all_reduce(self, arr: np.ndarray, average: bool = True, topk: int = 0) -> np.ndarray:
        assert arr.dtype == np.float32 and arr.flags["C_CONTIGUOUS"]
        fn = _lib().arix_dist_ring_all_reduce if average else None
        rc = fn(arr.ctypes.data, arr.size, topk) if average else _lib().arix_dist_all_reduce_sum(arr.ctypes.data, arr.size)
        if rc != 0:
            raise RuntimeError(f"ring all-reduce failed ({rc}): a peer closed its connection or timed out")
        return arr

    def sync_params(self, arr: np.ndarray, version: int) -> int:
        v = C.c_ulonglong(version)
        rc = _lib().arix_dist_sync_params(arr.ctypes.data, arr.size, C.byref(v))
        if rc != 0:
            raise RuntimeError(f"sync_params failed ({rc})")
        return v.value

    @staticmethod
    def add_noise(arr: np.ndarray, scale: float, seed: int = 0) -> np.ndarray:
        _lib().arix_dist_add_noise(arr.ctypes.data, arr.size, scale, seed)
        return arr

    def shutdown(self):
        _lib().arix_dist_shutdown()


class HeartbeatMonitor:
    """UDP heartbeats on port base + rank; peers late by more than ``timeout`` are SUSPECT, by more than three
    intervals (and the timeout) DEAD."""

    def __init__(self, rank: int, world: int, base_port: int = 28700, interval_s: float = 0.1, timeout_s: float = 0.5):
        self.rank, self.world = rank, world
        self._h = _lib().sx_hb_create(rank, world, base_port, int(interval_s * 1000), int(timeout_s * 1000))
        if not self._h:
            raise OSError("cannot bind heartbeat socket")
        self._started = False

    def start(self):
        _lib().sx_hb_start(self._h)
        self._started = True
        return self

    def status(self, rank: int) -> int:
        return _lib().sx_hb_status(self._h, rank)

    def alive_ranks(self) -> List[int]:
        return [r for r in range(self.world) if r == self.rank or self.status(r) != DEAD]

    def dead_ranks(self) -> List[int]:
        return [r for r in range(self.world) if r != self.rank and self.status(r) == DEAD]

    def pause_sending(self, paused: bool = True):
        """Host-side fault injection: this rank stops announcing itself (looks failed to its peers)."""
        _lib().sx_hb_set_send_enabled(self._h, 0 if paused else 1)

    def stop(self):
        if self._h:
            if self._started:
                _lib().sx_hb_stop(self._h)
            self._h = None


class ElasticMembership:
    """Rank table that grows on join and shrinks on leave / failure; refuses to drop below half of the original
    world or to remove itself; compacts ranks into a new dense topology."""

    def __init__(self, world: int, self_rank: int):
        self.original_world = world
        self.self_rank = self_rank
        self.members: List[int] = list(range(world))
        self.restarts = 0
        self.version = 0
        self.state = "ok"

    def join(self, rank: int) -> bool:
        if rank in self.members:
            return False
        self.members.append(rank)
        self.members.sort()
        self.version += 1
        return True

    def leave(self, rank: int) -> bool:
        if rank == self.self_rank or rank not in self.members:
            return False
        if (len(self.members) - 1) * 2 < self.original_world:
            return False
        self.members.remove(rank)
        self.version += 1
        return True

    def new_topology(self) -> Dict[int, int]:
        return {old: new for new, old in enumerate(self.members)}


class ElasticTrainer:
    """On a detected failure: bump the restart count (at most MAX_RESTARTS), drop the dead ranks, restore the last
    checkpoint (version - 1 when the current one may be partial) and re-form the topology after a barrier."""

    def __init__(self, membership: ElasticMembership, restore_fn: Callable[[int], bool],
                 barrier_fn: Optional[Callable[[], None]] = None):
        self.m, self.restore_fn, self.barrier_fn = membership, restore_fn, barrier_fn
        self.checkpoint_version = 0

    def mark_checkpoint(self, version: int):
        self.checkpoint_version = version

    def handle_failure(self, dead: List[int]) -> bool:
        if self.m.restarts >= MAX_RESTARTS:
            self.m.state = "failed"
            return False
        self.m.restarts += 1
        self.m.state = "recovering"
        for r in dead:
            if not self.m.leave(r):
                self.m.state = "failed"
                return False
        return self.reconfigure()

    def reconfigure(self) -> bool:
        if self.barrier_fn:
            self.barrier_fn()
        ok = self.restore_fn(max(self.checkpoint_version - 1, 0) if self.m.state == "recovering" and
                             self.checkpoint_version > 0 else self.checkpoint_version)
        self.m.state = "ok" if ok else "failed"
        return ok


class FaultToleranceManager:
    """Heartbeat + elastic trainer: ``poll()`` between steps returns the new rank mapping after a recovery."""

    def __init__(self, monitor: HeartbeatMonitor, trainer: ElasticTrainer):
        self.monitor, self.trainer = monitor, trainer
        self._handled = set()

    def poll(self):
        dead = [r for r in self.monitor.dead_ranks() if r not in self._handled]
        if not dead:
            return None
        self._handled.update(dead)
        if not self.trainer.handle_failure(dead):
            raise RuntimeError(f"unrecoverable failure of ranks {dead}")
        return self.trainer.m.new_topology()

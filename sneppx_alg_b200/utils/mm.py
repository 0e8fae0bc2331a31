"""Bindings of the C++ host memory managers and compression codecs (``csrc/host/mm.cpp``).

Reference counterparts: ``mm/arena``, ``mm/internal/slab_alloc.c`` (+ per-thread magazines), ``mm/internal/vmem.c``,
``mm/pool/object_pool.c``, ``mm/tiered/tiered_memory.c``, ``mm/huge/hugepage_mgr.c``, ``mm/internal/compress.c``.
Pointers are plain integers; ``view`` wraps one as a NumPy array without copying.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np

from .. import _build


def _L():
    L = _build.load_host()
    if not getattr(L, "_mm_ready", False):
        vp, ll, i = C.c_void_p, C.c_longlong, C.c_int
        sig = {
            "sx_arena_create": (vp, [ll]), "sx_arena_destroy": (None, [vp]), "sx_arena_alloc": (vp, [vp, ll]),
            "sx_arena_alloc_aligned": (vp, [vp, ll, ll]), "sx_arena_reset": (None, [vp]), "sx_arena_used": (ll, [vp]),
            "sx_arena_capacity": (ll, [vp]), "sx_arena_stats": (None, [vp, vp]),
            "sx_slab_create": (vp, [ll, i]), "sx_slab_destroy": (None, [vp]), "sx_slab_alloc": (vp, [vp]),
            "sx_slab_free": (i, [vp, vp]), "sx_slab_gc": (i, [vp]), "sx_slab_stats": (None, [vp, vp]),
            "sx_slab_local_create": (vp, [vp, i]), "sx_slab_local_alloc": (vp, [vp]), "sx_slab_local_free": (None, [vp, vp]),
            "sx_slab_local_flush": (None, [vp]), "sx_slab_local_destroy": (None, [vp]),
            "sx_vmem_page_size": (ll, []), "sx_vmem_reserve": (vp, [ll]), "sx_vmem_commit": (i, [vp, ll]),
            "sx_vmem_decommit": (i, [vp, ll]), "sx_vmem_release": (i, [vp, ll]), "sx_vmem_advise_hugepage": (i, [vp, ll, i]),
            "sx_objpool_create": (vp, [ll, i]), "sx_objpool_destroy": (None, [vp]), "sx_objpool_clear": (None, [vp]),
            "sx_objpool_prealloc": (i, [vp, i]), "sx_objpool_acquire": (vp, [vp]), "sx_objpool_release": (i, [vp, vp]),
            "sx_objpool_available": (i, [vp]), "sx_objpool_capacity": (i, [vp]),
            "sx_tiered_create": (vp, [vp, i, vp]), "sx_tiered_destroy": (None, [vp]), "sx_tiered_alloc": (vp, [vp, ll, i]),
            "sx_tiered_free": (i, [vp, vp]), "sx_tiered_migrate": (i, [vp, vp, i]), "sx_tiered_get_tier": (i, [vp, vp]),
            "sx_tiered_used": (ll, [vp, i]), "sx_tiered_name": (C.c_char_p, [vp, i]),
            "sx_compress_bound": (ll, [C.c_char_p, ll, i]),
            "sx_compress": (ll, [C.c_char_p, vp, ll, i, C.c_float, vp, ll]), "sx_decompress": (ll, [vp, ll, vp, ll]),
        }
        for name, (res, args) in sig.items():
            f = getattr(L, name)
            f.restype, f.argtypes = res, args
        L._mm_ready = True
    return L


def view(ptr: int, nbytes: int, dtype=np.uint8) -> np.ndarray:
    """NumPy view of `nbytes` at address `ptr` (no copy; the memory must outlive the array)."""
    buf = (C.c_char * nbytes).from_address(ptr)
    return np.frombuffer(buf, dtype=dtype)


class Arena:
    def __init__(self, chunk_size: int = 1 << 20):
        self._h = _L().sx_arena_create(chunk_size)

    def alloc(self, n: int, align: int = 16) -> int:
        p = _L().sx_arena_alloc_aligned(self._h, n, align)
        if not p:
            raise ValueError("alignment must be a power of two")
        return p

    def reset(self):
        _L().sx_arena_reset(self._h)

    def stats(self) -> dict:
        out = (C.c_longlong * 5)()
        _L().sx_arena_stats(self._h, out)
        return dict(zip(("used", "capacity", "chunks", "allocations", "peak"), out))

    def __del__(self):
        try:
            _L().sx_arena_destroy(self._h)
        except Exception:
            pass


class SlabCache:
    def __init__(self, obj_size: int, objs_per_slab: int = 64):
        self._h = _L().sx_slab_create(obj_size, objs_per_slab)

    def alloc(self) -> int:
        return _L().sx_slab_alloc(self._h)

    def free(self, p: int):
        if _L().sx_slab_free(self._h, p):
            raise ValueError("pointer does not belong to this cache")

    def gc(self) -> int:
        return _L().sx_slab_gc(self._h)

    def stats(self) -> dict:
        out = (C.c_longlong * 5)()
        _L().sx_slab_stats(self._h, out)
        return dict(zip(("slabs", "free", "allocations", "frees", "obj_size"), out))

    def magazine(self, size: int = 16) -> "Magazine":
        return Magazine(self, size)

    def __del__(self):
        try:
            _L().sx_slab_destroy(self._h)
        except Exception:
            pass


class Magazine:
    """Per-thread front end of a SlabCache: takes the cache lock once per half-magazine, not once per object."""

    def __init__(self, cache: SlabCache, size: int):
        self._cache = cache  # keeps the cache alive
        self._h = _L().sx_slab_local_create(cache._h, size)

    def alloc(self) -> int:
        return _L().sx_slab_local_alloc(self._h)

    def free(self, p: int):
        _L().sx_slab_local_free(self._h, p)

    def flush(self):
        _L().sx_slab_local_flush(self._h)

    def close(self):
        if self._h:
            _L().sx_slab_local_destroy(self._h)
            self._h = None


class VirtualRegion:
    """Address range reserved without backing; pages are committed and given back on demand."""

    def __init__(self, nbytes: int):
        self.page = _L().sx_vmem_page_size()
        self.size = (nbytes + self.page - 1) // self.page * self.page
        self.base = _L().sx_vmem_reserve(self.size)
        if not self.base:
            raise MemoryError("cannot reserve address space")

    def commit(self, offset: int, nbytes: int):
        if _L().sx_vmem_commit(self.base + offset, nbytes):
            raise MemoryError("commit failed")

    def decommit(self, offset: int, nbytes: int):
        if _L().sx_vmem_decommit(self.base + offset, nbytes):
            raise MemoryError("decommit failed")

    def advise_hugepage(self, on: bool = True) -> bool:
        return _L().sx_vmem_advise_hugepage(self.base, self.size, int(on)) == 0

    def release(self):
        if self.base:
            _L().sx_vmem_release(self.base, self.size)
            self.base = None


class ObjectPool:
    def __init__(self, obj_size: int, capacity: int, prealloc: int = 0):
        self._h = _L().sx_objpool_create(obj_size, capacity)
        if prealloc:
            _L().sx_objpool_prealloc(self._h, prealloc)

    def acquire(self) -> int:
        p = _L().sx_objpool_acquire(self._h)
        if not p:
            raise MemoryError("object pool exhausted")
        return p

    def release(self, p: int):
        rc = _L().sx_objpool_release(self._h, p)
        if rc:
            raise ValueError("foreign pointer" if rc == -1 else "double release")

    @property
    def available(self) -> int:
        return _L().sx_objpool_available(self._h)

    @property
    def capacity(self) -> int:
        return _L().sx_objpool_capacity(self._h)

    def __del__(self):
        try:
            _L().sx_objpool_destroy(self._h)
        except Exception:
            pass


class TieredMemory:
    """Capacity accounting over ordered tiers (fastest first) with fall-through allocation and migration."""

    def __init__(self, tier_sizes: Sequence[int], names: Sequence[str] | None = None):
        n = len(tier_sizes)
        sizes = (C.c_longlong * n)(*tier_sizes)
        nm = (C.c_char_p * n)(*[s.encode() for s in names]) if names else None
        self._h = _L().sx_tiered_create(sizes, n, nm)
        self.num_tiers = n

    def alloc(self, size: int, preferred_tier: int = 0) -> int:
        p = _L().sx_tiered_alloc(self._h, size, preferred_tier)
        if not p:
            raise MemoryError("no tier has room")
        return p

    def free(self, p: int):
        if _L().sx_tiered_free(self._h, p):
            raise ValueError("unknown block")

    def migrate(self, p: int, tier: int) -> bool:
        rc = _L().sx_tiered_migrate(self._h, p, tier)
        if rc == -1:
            raise ValueError("unknown block or tier")
        return rc == 0

    def tier_of(self, p: int) -> int:
        return _L().sx_tiered_get_tier(self._h, p)

    def used(self, tier: int) -> int:
        return _L().sx_tiered_used(self._h, tier)

    def name(self, tier: int) -> str:
        return _L().sx_tiered_name(self._h, tier).decode()

    def __del__(self):
        try:
            _L().sx_tiered_destroy(self._h)
        except Exception:
            pass


CODECS = ("none", "bfp8", "bfp4", "sparse")


def compress(x: np.ndarray, codec: str = "bfp8", block: int = 32, threshold: float = 0.0) -> bytes:
    """fp32 array -> byte stream (see the stream layout in ``csrc/host/mm.cpp``)."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    cap = _L().sx_compress_bound(codec.encode(), x.size, block)
    if cap < 0:
        raise KeyError(f"unknown codec {codec!r}; have {CODECS}")
    out = C.create_string_buffer(cap)
    n = _L().sx_compress(codec.encode(), x.ctypes.data, x.size, block, threshold, out, cap)
    if n < 0:
        raise RuntimeError(f"compress failed ({n})")
    return out.raw[:n]


def decompress(stream: bytes, n: int) -> np.ndarray:
    y = np.empty(n, dtype=np.float32)
    got = _L().sx_decompress(stream, len(stream), y.ctypes.data, n)
    if got < 0:
        raise ValueError("malformed stream or short output buffer")
    return y[:got]

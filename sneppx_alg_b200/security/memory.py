"""S1 secure memory and S3 in-process tamper monitors: Python face of ``csrc/host/memsec.cpp``.

``LeakDetector`` (tracked allocations with call sites, threshold, report), ``Quarantine`` (freed blocks poisoned and
parked; writes to a parked block are reported as use after free), ``PointerAuth`` (keyed pointer tags),
``ControlFlowGuard`` (allowed indirect-call targets), ``ShadowStack``, ``CanaryPool``, ``GuardPagePool`` (allocations
fenced by inaccessible pages), ``MemoryPressure`` (soft / hard byte budget), ``mask_metadata``, ``CodeTamperDetector``
(digests of memory regions), ``HeapSentinels`` and ``set_memory_mode`` (W^X). The reference's modules of the same
purpose: security/memory/memory_leak_detector.c, security/memory/memory_hardening.c,
security/monitor/monitor_advanced.c."""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

from .. import _build


def _L():
    L = _build.load_host()
    if not getattr(L, "_memsec_ready", False):
        for f in ("sx_leak_malloc", "sx_leak_realloc", "sx_quarantine_create", "sx_pac_create", "sx_cfg_create",
                  "sx_shadow_create", "sx_canary_pool_create", "sx_guard_pool_create", "sx_guard_pool_alloc",
                  "sx_mem_alloc_pages", "sx_pressure_create"):
            getattr(L, f).restype = C.c_void_p
        L.sx_leak_malloc.argtypes = [C.c_size_t, C.c_char_p, C.c_int, C.c_char_p]
        L.sx_leak_realloc.argtypes = [C.c_void_p, C.c_size_t, C.c_char_p, C.c_int, C.c_char_p]
        L.sx_leak_free.argtypes = [C.c_void_p]
        L.sx_leak_free.restype = None
        L.sx_leak_track_alloc.argtypes = [C.c_void_p, C.c_size_t, C.c_char_p, C.c_int, C.c_char_p]
        L.sx_leak_track_free.argtypes = [C.c_void_p]
        L.sx_leak_check.argtypes = [C.c_char_p, C.c_size_t]
        L.sx_leak_stats.argtypes = [C.c_void_p]
        L.sx_leak_set_threshold.argtypes = [C.c_longlong]
        L.sx_quarantine_create.argtypes = [C.c_size_t]
        L.sx_quarantine_add.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        L.sx_quarantine_contains.argtypes = [C.c_void_p, C.c_void_p]
        L.sx_quarantine_stats.argtypes = [C.c_void_p, C.c_void_p]
        for f in ("sx_quarantine_drain", "sx_quarantine_destroy", "sx_pac_destroy", "sx_cfg_destroy", "sx_shadow_destroy",
                  "sx_canary_pool_destroy", "sx_guard_pool_destroy", "sx_pressure_destroy"):
            getattr(L, f).argtypes = [C.c_void_p]
        L.sx_pac_sign.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.sx_pac_sign.restype = C.c_ulonglong
        L.sx_pac_verify.argtypes = [C.c_void_p, C.c_void_p, C.c_ulonglong, C.c_int]
        L.sx_cfg_add_target.argtypes = L.sx_cfg_validate.argtypes = [C.c_void_p, C.c_void_p]
        L.sx_cfg_violations.argtypes = [C.c_void_p]
        L.sx_cfg_violations.restype = C.c_longlong
        L.sx_shadow_create.argtypes = [C.c_size_t]
        L.sx_shadow_push.argtypes = L.sx_shadow_pop_check.argtypes = [C.c_void_p, C.c_ulonglong]
        L.sx_shadow_depth.argtypes = [C.c_void_p]
        L.sx_shadow_depth.restype = C.c_longlong
        L.sx_canary_alloc.argtypes = [C.c_void_p]
        L.sx_canary_alloc.restype = C.c_ulonglong
        L.sx_canary_check.argtypes = [C.c_void_p, C.c_ulonglong]
        L.sx_guard_pool_alloc.argtypes = [C.c_void_p, C.c_size_t]
        L.sx_guard_pool_free.argtypes = [C.c_void_p, C.c_void_p]
        L.sx_guard_pool_room.argtypes = [C.c_void_p, C.c_void_p]
        L.sx_guard_pool_room.restype = C.c_longlong
        L.sx_guard_pool_live.argtypes = [C.c_void_p]
        L.sx_guard_pool_live.restype = C.c_longlong
        L.sx_mem_set_mode.argtypes = [C.c_void_p, C.c_size_t, C.c_int]
        L.sx_mem_alloc_pages.argtypes = [C.c_size_t]
        L.sx_mem_free_pages.argtypes = [C.c_void_p, C.c_size_t]
        L.sx_pressure_create.argtypes = [C.c_longlong, C.c_longlong]
        L.sx_pressure_reserve.argtypes = [C.c_void_p, C.c_longlong]
        L.sx_pressure_release.argtypes = [C.c_void_p, C.c_longlong]
        L.sx_pressure_release.restype = None
        for f in ("sx_pressure_used", "sx_pressure_rejected"):
            getattr(L, f).argtypes = [C.c_void_p]
            getattr(L, f).restype = C.c_longlong
        L.sx_metadata_mask.argtypes = [C.c_char_p, C.c_void_p, C.c_size_t, C.c_ulonglong]
        L.sx_metadata_mask.restype = None
        L.sx_tamper_add_region.argtypes = [C.c_void_p, C.c_size_t]
        L.sx_sentinel_apply.argtypes = [C.c_void_p, C.c_size_t]
        L.sx_sentinel_apply.restype = None
        L.sx_sentinel_check.argtypes = [C.c_void_p, C.c_size_t]
        L.sx_sentinel_set_value.argtypes = [C.c_ulonglong]
        L.sx_sentinel_set_value.restype = None
        L._memsec_ready = True
    return L


class LeakDetector:
    """Process-wide allocation tracker. ``malloc`` / ``free`` allocate through it; ``track`` / ``untrack`` register
    memory obtained elsewhere."""

    def __init__(self, threshold: int = 0):
        _L().sx_leak_reset()
        _L().sx_leak_enable(1)
        _L().sx_leak_set_threshold(threshold)

    def malloc(self, n: int, file: str = "", line: int = 0, func: str = "") -> int:
        return _L().sx_leak_malloc(n, file.encode(), line, func.encode()) or 0

    def realloc(self, p: int, n: int, file: str = "", line: int = 0, func: str = "") -> int:
        return _L().sx_leak_realloc(p, n, file.encode(), line, func.encode()) or 0

    def free(self, p: int) -> None:
        _L().sx_leak_free(p)

    def track(self, p: int, n: int, file: str = "", line: int = 0, func: str = "") -> None:
        _L().sx_leak_track_alloc(p, n, file.encode(), line, func.encode())

    def untrack(self, p: int) -> bool:
        """False when the pointer was not tracked (double free or foreign pointer)."""
        return _L().sx_leak_track_free(p) == 0

    def set_threshold(self, n: int) -> None:
        _L().sx_leak_set_threshold(n)

    def enable(self, on: bool = True) -> None:
        _L().sx_leak_enable(int(on))

    def stats(self) -> dict:
        out = (C.c_longlong * 7)()
        _L().sx_leak_stats(out)
        keys = ("live_blocks", "live_bytes", "peak_bytes", "total_bytes", "allocations", "frees", "unknown_frees")
        return dict(zip(keys, (int(v) for v in out)))

    def report(self) -> List[dict]:
        """Live blocks at or above the threshold, oldest first."""
        buf = C.create_string_buffer(1 << 16)
        _L().sx_leak_check(buf, len(buf))
        out = []
        for line in buf.value.decode().splitlines():
            seq, size, where, func = (line.split(" ", 3) + [""])[:4]
            file, _, ln = where.rpartition(":")
            out.append({"seq": int(seq), "size": int(size), "file": file, "line": int(ln or 0), "func": func})
        return out

    def reset(self) -> None:
        _L().sx_leak_reset()


class Quarantine:
    def __init__(self, budget_bytes: int = 1 << 20):
        self._h = _L().sx_quarantine_create(budget_bytes)
        self._libc = C.CDLL(None)
        self._libc.malloc.restype = C.c_void_p
        self._libc.malloc.argtypes = [C.c_size_t]

    def malloc(self, n: int) -> int:
        return self._libc.malloc(n)

    def retire(self, p: int, n: int) -> int:
        """Park a block instead of freeing it; returns how many use-after-free writes were found in blocks that left
        the quarantine because of this call."""
        return _L().sx_quarantine_add(self._h, p, n)

    def is_dangling(self, p: int) -> bool:
        return bool(_L().sx_quarantine_contains(self._h, p))

    def stats(self) -> dict:
        out = (C.c_longlong * 4)()
        _L().sx_quarantine_stats(self._h, out)
        return dict(zip(("parked_blocks", "parked_bytes", "released", "use_after_free"), (int(v) for v in out)))

    def drain(self) -> int:
        return _L().sx_quarantine_drain(self._h)

    def close(self) -> None:
        if self._h:
            _L().sx_quarantine_destroy(self._h)
            self._h = None


class PointerAuth:
    def __init__(self):
        self._h = _L().sx_pac_create()

    def sign(self, pointer: int, key: int = 0) -> int:
        return int(_L().sx_pac_sign(self._h, pointer, key))

    def verify(self, pointer: int, tag: int, key: int = 0) -> bool:
        return bool(_L().sx_pac_verify(self._h, pointer, tag, key))


class ControlFlowGuard:
    def __init__(self):
        self._h = _L().sx_cfg_create()

    def allow(self, target: int) -> None:
        _L().sx_cfg_add_target(self._h, target)

    def validate(self, target: int) -> bool:
        return bool(_L().sx_cfg_validate(self._h, target))

    @property
    def violations(self) -> int:
        return int(_L().sx_cfg_violations(self._h))


class ShadowStack:
    def __init__(self, capacity: int = 4096):
        self._h = _L().sx_shadow_create(capacity)

    def push(self, return_address: int) -> None:
        if _L().sx_shadow_push(self._h, return_address) != 0:
            raise OverflowError("shadow stack is full")

    def pop_check(self, return_address: int) -> bool:
        r = _L().sx_shadow_pop_check(self._h, return_address)
        if r < 0:
            raise IndexError("shadow stack is empty")
        return r == 1

    def __len__(self):
        return int(_L().sx_shadow_depth(self._h))


class CanaryPool:
    def __init__(self):
        self._h = _L().sx_canary_pool_create()

    def alloc(self) -> int:
        return int(_L().sx_canary_alloc(self._h))

    def check(self, canary: int) -> bool:
        return bool(_L().sx_canary_check(self._h, canary))


class GuardPagePool:
    """Allocations with an inaccessible page on both sides; ``room(p)`` is the distance from p to the guard."""

    def __init__(self):
        self._h = _L().sx_guard_pool_create()

    def alloc(self, n: int) -> int:
        p = _L().sx_guard_pool_alloc(self._h, n)
        if not p:
            raise MemoryError("guard pool allocation failed")
        return p

    def room(self, p: int) -> int:
        return int(_L().sx_guard_pool_room(self._h, p))

    def free(self, p: int) -> bool:
        return _L().sx_guard_pool_free(self._h, p) == 0

    @property
    def live(self) -> int:
        return int(_L().sx_guard_pool_live(self._h))

    def close(self) -> None:
        if self._h:
            _L().sx_guard_pool_destroy(self._h)
            self._h = None


class MemoryPressure:
    OK, SOFT, REJECTED = 0, 1, -1

    def __init__(self, soft_limit: int, hard_limit: int):
        self._h = _L().sx_pressure_create(soft_limit, hard_limit)

    def reserve(self, n: int) -> int:
        return _L().sx_pressure_reserve(self._h, n)

    def release(self, n: int) -> None:
        _L().sx_pressure_release(self._h, n)

    @property
    def used(self) -> int:
        return int(_L().sx_pressure_used(self._h))

    @property
    def rejected(self) -> int:
        return int(_L().sx_pressure_rejected(self._h))


def mask_metadata(key16: bytes, data: bytes, tweak: int = 0) -> bytes:
    """XOR mask of allocator metadata kept in memory (the same call unmasks)."""
    assert len(key16) == 16
    buf = C.create_string_buffer(bytes(data), len(data))
    _L().sx_metadata_mask(key16, buf, len(data), tweak)
    return buf.raw


def set_memory_mode(addr: int, n: int, executable: bool) -> bool:
    """W^X: a page range is either writable or executable, never both."""
    return _L().sx_mem_set_mode(addr, n, int(executable)) == 0


def alloc_pages(n: int) -> int:
    return _L().sx_mem_alloc_pages(n) or 0


def free_pages(p: int, n: int) -> None:
    _L().sx_mem_free_pages(p, n)


class CodeTamperDetector:
    def __init__(self):
        self.regions: List[int] = []
        self._keep = []

    def add_buffer(self, buf) -> int:
        """Watch a ctypes buffer / bytearray-backed ctypes array."""
        self._keep.append(buf)
        i = _L().sx_tamper_add_region(C.addressof(buf), C.sizeof(buf))
        self.regions.append(i)
        return i

    def add_region(self, addr: int, n: int) -> int:
        i = _L().sx_tamper_add_region(addr, n)
        self.regions.append(i)
        return i

    def check(self, i: int) -> Optional[bool]:
        r = _L().sx_tamper_check(i)
        return None if r < 0 else bool(r)

    def remove(self, i: int) -> bool:
        return _L().sx_tamper_remove_region(i) == 0

    def modified_regions(self) -> int:
        return int(_L().sx_tamper_check_all())


class HeapSentinels:
    def __init__(self, value: Optional[int] = None):
        if value is not None:
            _L().sx_sentinel_set_value(value)

    def apply(self, addr: int, n: int) -> None:
        _L().sx_sentinel_apply(addr, n)

    def intact(self, addr: int, n: int) -> bool:
        return bool(_L().sx_sentinel_check(addr, n))

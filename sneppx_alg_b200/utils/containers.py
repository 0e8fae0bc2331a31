"""Python face of the host runtime's containers (``csrc/host/containers.cpp``): ``HashTable`` (64-bit keys),
``PriorityQueue`` (smallest first, FIFO among equals), ``RBTree`` (ordered keys with successor / predecessor queries)
and string helpers. Values are unsigned 64-bit words. Reference: lib/internal/{hashtable,pqueue,rbtree,strutil}.c."""
from __future__ import annotations

import ctypes as C
from typing import Iterator, List, Optional, Tuple

from .. import _build

_VISIT = C.CFUNCTYPE(None, C.c_ulonglong, C.c_ulonglong, C.c_void_p)


def _L():
    L = _build.load_host()
    if not getattr(L, "_ct_ready", False):
        for f in ("sx_ht_create", "sx_pq_create", "sx_rbtree_create", "sx_strbuf_create"):
            getattr(L, f).restype = C.c_void_p
        L.sx_ht_create.argtypes = L.sx_pq_create.argtypes = L.sx_strbuf_create.argtypes = [C.c_size_t]
        u64, p64 = C.c_ulonglong, C.POINTER(C.c_ulonglong)
        L.sx_ht_insert.argtypes = L.sx_pq_push.argtypes = L.sx_rbtree_insert.argtypes = [C.c_void_p, u64, u64]
        L.sx_ht_lookup.argtypes = L.sx_rbtree_search.argtypes = [C.c_void_p, u64, p64]
        L.sx_ht_delete.argtypes = L.sx_rbtree_delete.argtypes = [C.c_void_p, u64]
        L.sx_pq_pop.argtypes = L.sx_pq_peek.argtypes = [C.c_void_p, p64, p64]
        L.sx_rbtree_min.argtypes = L.sx_rbtree_max.argtypes = [C.c_void_p, p64]
        L.sx_rbtree_successor.argtypes = L.sx_rbtree_predecessor.argtypes = [C.c_void_p, u64, p64]
        L.sx_ht_foreach.argtypes = L.sx_rbtree_foreach.argtypes = [C.c_void_p, _VISIT, C.c_void_p]
        L.sx_ht_resize.argtypes = [C.c_void_p, C.c_size_t]
        for f in ("sx_ht_size", "sx_ht_capacity", "sx_pq_size", "sx_rbtree_size", "sx_strbuf_length"):
            getattr(L, f).argtypes = [C.c_void_p]
            getattr(L, f).restype = C.c_size_t
        for f in ("sx_ht_destroy", "sx_ht_clear", "sx_pq_destroy", "sx_pq_clear", "sx_rbtree_destroy", "sx_strbuf_destroy",
                  "sx_strbuf_clear", "sx_ht_max_probe", "sx_pq_is_empty", "sx_rbtree_validate"):
            getattr(L, f).argtypes = [C.c_void_p]
        L.sx_strbuf_append.argtypes = [C.c_void_p, C.c_char_p]
        L.sx_strbuf_cstr.argtypes = [C.c_void_p]
        L.sx_strbuf_cstr.restype = C.c_char_p
        L.sx_strlcpy.argtypes = L.sx_strlcat.argtypes = [C.c_char_p, C.c_char_p, C.c_size_t]
        L.sx_strlcpy.restype = L.sx_strlcat.restype = C.c_size_t
        L.sx_strsplit.argtypes = [C.c_char_p, C.c_char, C.c_char_p, C.c_size_t, C.c_size_t]
        L.sx_strsplit.restype = C.c_longlong
        L._ct_ready = True
    return L


def _collect(fn, handle) -> List[Tuple[int, int]]:
    out: List[Tuple[int, int]] = []
    cb = _VISIT(lambda k, v, _c: out.append((int(k), int(v))))
    fn(handle, cb, None)
    return out


class HashTable:
    def __init__(self, capacity: int = 16):
        self._h = _L().sx_ht_create(capacity)

    def __setitem__(self, key: int, value: int) -> None:
        _L().sx_ht_insert(self._h, key, value)

    def get(self, key: int, default=None):
        v = C.c_ulonglong()
        return int(v.value) if _L().sx_ht_lookup(self._h, key, C.byref(v)) else default

    def __getitem__(self, key: int) -> int:
        v = self.get(key)
        if v is None:
            raise KeyError(key)
        return v

    def __contains__(self, key: int) -> bool:
        return bool(_L().sx_ht_lookup(self._h, key, None))

    def __delitem__(self, key: int) -> None:
        if not _L().sx_ht_delete(self._h, key):
            raise KeyError(key)

    def __len__(self) -> int:
        return int(_L().sx_ht_size(self._h))

    @property
    def capacity(self) -> int:
        return int(_L().sx_ht_capacity(self._h))

    @property
    def max_probe(self) -> int:
        return int(_L().sx_ht_max_probe(self._h))

    def items(self) -> List[Tuple[int, int]]:
        return _collect(_L().sx_ht_foreach, self._h)

    def clear(self) -> None:
        _L().sx_ht_clear(self._h)

    def resize(self, capacity: int) -> bool:
        return _L().sx_ht_resize(self._h, capacity) == 0

    def __del__(self):
        try:
            _L().sx_ht_destroy(self._h)
        except Exception:  # noqa: BLE001
            pass


class PriorityQueue:
    def __init__(self, capacity: int = 16):
        self._h = _L().sx_pq_create(capacity)

    def push(self, priority: int, value: int) -> None:
        _L().sx_pq_push(self._h, priority, value)

    def _take(self, fn) -> Optional[Tuple[int, int]]:
        p, v = C.c_ulonglong(), C.c_ulonglong()
        return (int(p.value), int(v.value)) if fn(self._h, C.byref(p), C.byref(v)) else None

    def pop(self) -> Optional[Tuple[int, int]]:
        return self._take(_L().sx_pq_pop)

    def peek(self) -> Optional[Tuple[int, int]]:
        return self._take(_L().sx_pq_peek)

    def __len__(self) -> int:
        return int(_L().sx_pq_size(self._h))

    def clear(self) -> None:
        _L().sx_pq_clear(self._h)

    def __del__(self):
        try:
            _L().sx_pq_destroy(self._h)
        except Exception:  # noqa: BLE001
            pass


class RBTree:
    def __init__(self):
        self._h = _L().sx_rbtree_create()

    def insert(self, key: int, value: int = 0) -> bool:
        """True when the key is new."""
        return _L().sx_rbtree_insert(self._h, key, value) == 0

    def search(self, key: int, default=None):
        v = C.c_ulonglong()
        return int(v.value) if _L().sx_rbtree_search(self._h, key, C.byref(v)) else default

    def delete(self, key: int) -> bool:
        return bool(_L().sx_rbtree_delete(self._h, key))

    def _q(self, fn, *a) -> Optional[int]:
        v = C.c_ulonglong()
        return int(v.value) if fn(self._h, *a, C.byref(v)) else None

    def min(self) -> Optional[int]:
        return self._q(_L().sx_rbtree_min)

    def max(self) -> Optional[int]:
        return self._q(_L().sx_rbtree_max)

    def successor(self, key: int) -> Optional[int]:
        return self._q(_L().sx_rbtree_successor, key)

    def predecessor(self, key: int) -> Optional[int]:
        return self._q(_L().sx_rbtree_predecessor, key)

    def items(self) -> List[Tuple[int, int]]:
        return _collect(_L().sx_rbtree_foreach, self._h)

    def __len__(self) -> int:
        return int(_L().sx_rbtree_size(self._h))

    def black_height(self) -> int:
        """>= 1 when every red-black and ordering rule holds, -1 otherwise."""
        return int(_L().sx_rbtree_validate(self._h))

    def __del__(self):
        try:
            _L().sx_rbtree_destroy(self._h)
        except Exception:  # noqa: BLE001
            pass


def strlcpy(src: str, cap: int) -> Tuple[str, int]:
    """(what fits into a buffer of ``cap`` bytes, length the source needed)."""
    buf = C.create_string_buffer(max(cap, 1))
    n = _L().sx_strlcpy(buf, src.encode(), cap)
    return buf.value.decode(errors="ignore"), int(n)


def strsplit(s: str, delim: str, max_tokens: int = 0) -> List[str]:
    raw = s.encode()
    buf = C.create_string_buffer(len(raw) + s.count(delim) + 2)
    n = _L().sx_strsplit(raw, delim.encode(), buf, len(buf), max_tokens)
    if n < 0:
        raise MemoryError("token buffer too small")
    return [t.decode() for t in buf.raw.split(b"\x00")[: int(n)]]

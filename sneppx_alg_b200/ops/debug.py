"""Debug-bounds mode (``SX_DEBUG_BOUNDS=1`` or ``enable()``): the checks a memory sanitizer would give, built so
that nothing ever faults or traps on the GPU.

* every index array that drives a gather / scatter kernel (MoE slots and row -> token maps, tile -> expert tables,
  paged-KV block tables and slot maps, loss targets, expert-dispatch destinations) is range-checked by a small
  kernel before the consuming kernel is launched; the first bad value is recorded on the device
  (site, position, value, limits) and ``check()`` raises ``KernelBoundsError`` from it;
* outputs are pre-filled with a NaN pattern (``poison_``), so an element a kernel failed to write is visible in
  the result instead of silently holding stale data;
* symmetric (peer-mapped) buffers get guard zones on both sides filled with a canary pattern that
  ``SymmGroup.check_canaries()`` verifies (``parallel/symm.py``).

The reference's counterparts are a device ``assert`` macro under ``SNEPPX_DEBUG`` (kernel/cuda/common.cuh:172-181)
and a sanitizer script (scripts/run_sanitizers.sh:15-73); a device assert kills the context, which this mode avoids.
Off by default: the checks cost extra launches and one synchronising read per ``check()``.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import _lib

ENABLED = os.environ.get("SX_DEBUG_BOUNDS", "0") == "1"

SITE_MOE_SLOT, SITE_MOE_ROW_TOKEN, SITE_TILE_GROUP, SITE_BLOCK_TABLE, SITE_KV_SLOT, SITE_CE_TARGET, SITE_EP_ROW, \
    SITE_EP_RANK, SITE_USER = range(1, 10)
SITE_NAMES = {SITE_MOE_SLOT: "MoE slot of a routed entry", SITE_MOE_ROW_TOKEN: "MoE row -> token map",
              SITE_TILE_GROUP: "grouped GEMM tile -> expert table", SITE_BLOCK_TABLE: "paged-KV block table",
              SITE_KV_SLOT: "KV append slot map", SITE_CE_TARGET: "cross-entropy target",
              SITE_EP_ROW: "expert-parallel destination row", SITE_EP_RANK: "expert-parallel destination rank",
              SITE_USER: "caller-defined"}


class KernelBoundsError(RuntimeError):
    """An index array held a value outside its range; the kernel that would have used it was not trusted."""


def enable(flag: bool = True) -> None:
    global ENABLED
    ENABLED = bool(flag)


def _active(t) -> bool:
    return ENABLED and torch.is_tensor(t) and t.is_cuda and _lib.available()


def check_indices(t, lo: int, hi: int, site: int, also_ok=None) -> None:
    """Queue a range check of an int32 / int64 index tensor: every value in [lo, hi) (or equal to ``also_ok``)."""
    if not _active(t) or t.numel() == 0:
        return
    t = t.contiguous()
    if t.dtype == torch.int32 and also_ok is None:
        _lib.call("sx_debug_check_indices", _lib.ptr(t), C.c_longlong(t.numel()), C.c_longlong(lo), C.c_longlong(hi),
                  C.c_int(site), _lib.stream())
    else:
        t64 = t if t.dtype == torch.int64 else t.long()
        _lib.call("sx_debug_check_indices64", _lib.ptr(t64), C.c_longlong(t64.numel()), C.c_longlong(lo), C.c_longlong(hi),
                  C.c_longlong(lo if also_ok is None else also_ok), C.c_int(site), _lib.stream())


def poison_(t) -> None:
    """Fill a freshly allocated output with NaNs (bf16 / fp16 / fp32 tensors whose byte size is a multiple of 4)."""
    if not _active(t) or t.numel() == 0 or not t.is_contiguous():
        return
    nbytes = t.numel() * t.element_size()
    if nbytes % 4 or t.dtype not in (torch.bfloat16, torch.float16, torch.float32):
        return
    pattern = {torch.bfloat16: 0x7FC07FC0, torch.float16: 0x7E007E00, torch.float32: 0x7FC00000}[t.dtype]
    _lib.call("sx_debug_poison", _lib.ptr(t), C.c_longlong(nbytes), C.c_uint(pattern), _lib.stream())


def read_record(reset: bool = True):
    """(site, position, value, lo, hi) of the first recorded violation, or None. Synchronises the device."""
    if not (torch.cuda.is_available() and _lib.available()):
        return None
    out = (C.c_longlong * 5)()
    torch.cuda.synchronize()
    rc = _lib.lib().sx_debug_record_read(out, C.c_int(int(reset)))
    if rc != 0:
        raise RuntimeError(f"sx_debug_record_read failed with code {rc}")
    return None if out[0] == 0 else tuple(int(v) for v in out)


def check() -> None:
    rec = read_record()
    if rec is not None:
        site, pos, val, lo, hi = rec
        raise KernelBoundsError(f"{SITE_NAMES.get(site, f'site {site}')}: element {pos} is {val}, outside [{lo}, {hi})")

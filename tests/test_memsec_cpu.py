"""Secure-memory layer and tamper monitors (native): leak reports, use-after-free detection in the quarantine, pointer
tags, control-flow set, shadow stack, canaries, guard pages, memory pressure, metadata masking, code-tamper digests,
heap sentinels, W^X."""
import ctypes as C

import pytest

from sneppx_alg_b200.security import memory as m


def test_leak_detector_reports_call_sites_and_unknown_frees():
    d = m.LeakDetector()
    a = d.malloc(100, "model.c", 10, "load")
    b = d.malloc(5000, "cache.c", 77, "fill")
    c = d.malloc(64, "tmp.c", 3, "scratch")
    d.free(c)
    st = d.stats()
    assert st["live_blocks"] == 2 and st["live_bytes"] == 5100 and st["peak_bytes"] == 5164 and st["frees"] == 1
    rep = d.report()
    assert [(r["file"], r["line"], r["func"], r["size"]) for r in rep] == [("model.c", 10, "load", 100), ("cache.c", 77, "fill", 5000)]
    d.set_threshold(1000)
    assert [r["size"] for r in d.report()] == [5000]
    b = d.realloc(b, 9000, "cache.c", 80, "grow")
    assert d.stats()["live_bytes"] == 9100
    d.free(a)
    d.free(b)
    assert d.stats()["live_blocks"] == 0
    assert d.untrack(0x1234) is False and d.stats()["unknown_frees"] == 1


def test_quarantine_detects_write_after_free():
    q = m.Quarantine(budget_bytes=300)
    p1, p2 = q.malloc(128), q.malloc(128)
    assert q.retire(p1, 128) == 0 and q.is_dangling(p1 + 5) and not q.is_dangling(p2)
    assert C.string_at(p1, 4) == b"\xdd" * 4                 # poisoned
    C.memset(p1 + 10, 0x41, 1)                               # a write through the dangling pointer
    assert q.retire(p2, 128) == 0                            # still within the budget
    p3 = q.malloc(128)
    assert q.retire(p3, 128) == 1                            # p1 leaves the quarantine: its damage is reported
    st = q.stats()
    assert st["use_after_free"] == 1 and st["released"] == 1 and st["parked_blocks"] == 2
    assert q.drain() == 0
    q.close()


def test_pointer_tags_cfg_shadow_stack_canaries():
    pa = m.PointerAuth()
    t = pa.sign(0x7F0012345678, 1)
    assert pa.verify(0x7F0012345678, t, 1)
    assert not pa.verify(0x7F0012345679, t, 1) and not pa.verify(0x7F0012345678, t, 2) and not pa.verify(0x7F0012345678, t ^ 1, 1)
    assert m.PointerAuth().sign(0x7F0012345678, 1) != t      # per-instance keys
    cfg = m.ControlFlowGuard()
    cfg.allow(0x1000)
    assert cfg.validate(0x1000) and not cfg.validate(0x1008) and cfg.violations == 1
    ss = m.ShadowStack(2)
    ss.push(0xAAA)
    ss.push(0xBBB)
    with pytest.raises(OverflowError):
        ss.push(0xCCC)
    assert ss.pop_check(0xBBB) and not ss.pop_check(0xDEAD) and len(ss) == 0
    with pytest.raises(IndexError):
        ss.pop_check(1)
    cp = m.CanaryPool()
    c1, c2 = cp.alloc(), cp.alloc()
    assert c1 != c2 and c1 & 0xFF == 0 and cp.check(c1) and not cp.check(c1) and not cp.check(c2 ^ 0x100) and cp.check(c2)


def test_guard_pages_pressure_masking():
    gp = m.GuardPagePool()
    p = gp.alloc(1000)
    assert p % 16 == 0 and 1000 <= gp.room(p) < 1016          # the block ends (almost) flush against the guard page
    C.memset(p, 0x55, 1000)
    assert gp.live == 1 and gp.free(p) and not gp.free(p) and gp.live == 0
    gp.close()
    mp = m.MemoryPressure(soft_limit=1000, hard_limit=2000)
    assert mp.reserve(900) == mp.OK and mp.reserve(500) == mp.SOFT and mp.reserve(700) == mp.REJECTED
    assert mp.used == 1400 and mp.rejected == 1
    mp.release(1400)
    assert mp.used == 0
    key = bytes(range(16))
    meta = b"size=4096;next=0x7f00;flags=3"
    masked = m.mask_metadata(key, meta, tweak=0x7F00)
    assert masked != meta and m.mask_metadata(key, masked, tweak=0x7F00) == meta
    assert m.mask_metadata(key, meta, tweak=0x7F08) != masked


def test_tamper_digests_sentinels_and_wx():
    det = m.CodeTamperDetector()
    code = C.create_string_buffer(b"\x90" * 256, 256)
    i = det.add_buffer(code)
    assert det.check(i) is True and det.modified_regions() == 0
    code[17] = b"\xcc"
    assert det.check(i) is False and det.modified_regions() == 1
    assert det.remove(i) and det.check(i) is None
    hs = m.HeapSentinels()
    buf = C.create_string_buffer(64 + 8)
    hs.apply(C.addressof(buf), 64)
    assert hs.intact(C.addressof(buf), 64)
    C.memset(C.addressof(buf) + 60, 0x41, 8)                 # an overflow of 4 bytes past the user range
    assert not hs.intact(C.addressof(buf), 64)
    page = m.alloc_pages(4096)
    assert page and m.set_memory_mode(page, 4096, executable=True) and m.set_memory_mode(page, 4096, executable=False)
    C.memset(page, 0, 16)                                     # writable again
    assert not m.set_memory_mode(page + 8, 4096, executable=True)   # unaligned range is refused
    m.free_pages(page, 4096)

"""C++ host allocators and compression codecs."""
import numpy as np
import pytest

from sneppx_alg_b200.utils import mm


def test_arena_alignment_growth_reset():
    a = mm.Arena(chunk_size=8192)
    p1 = a.alloc(100, 64)
    p2 = a.alloc(100, 256)
    assert p1 % 64 == 0 and p2 % 256 == 0 and p2 >= p1 + 100
    mm.view(p1, 100)[:] = 7
    big = a.alloc(100000, 4096)  # larger than a chunk: gets a chunk of its own
    assert big % 4096 == 0
    mm.view(big, 100000)[:] = 1
    st = a.stats()
    assert st["chunks"] == 2 and st["allocations"] == 3 and st["used"] >= 100200
    with pytest.raises(ValueError):
        a.alloc(8, 24)
    a.reset()
    st = a.stats()
    assert st["used"] == 0 and st["chunks"] == 1 and st["peak"] >= 100200


def test_slab_cache_reuse_gc_and_magazine():
    c = mm.SlabCache(48, objs_per_slab=8)
    ptrs = [c.alloc() for _ in range(20)]
    assert len(set(ptrs)) == 20 and c.stats()["slabs"] == 3 and c.stats()["obj_size"] == 48
    for p in ptrs:
        c.free(p)
    assert c.alloc() in ptrs  # reuse, no new slab
    assert c.gc() == 2 and c.stats()["slabs"] == 1
    with pytest.raises(ValueError):
        c.free(12345)
    m = c.magazine(size=8)
    got = [m.alloc() for _ in range(10)]
    assert len(set(got)) == 10
    for p in got:
        m.free(p)
    m.flush()
    st = c.stats()
    assert st["allocations"] - st["frees"] == 1  # only the object taken above is still out
    m.close()


def test_virtual_region_commit_decommit():
    r = mm.VirtualRegion(1 << 24)
    r.commit(0, 2 * r.page)
    v = mm.view(r.base, 2 * r.page)
    v[:] = 5
    assert int(v.sum()) == 10 * r.page
    r.decommit(r.page, r.page)
    r.commit(r.page, r.page)
    assert int(mm.view(r.base + r.page, r.page).sum()) == 0  # decommitted pages come back zeroed
    assert int(mm.view(r.base, r.page).sum()) == 5 * r.page
    r.advise_hugepage(True)
    r.release()


def test_object_pool_bounds():
    p = mm.ObjectPool(64, capacity=3, prealloc=2)
    assert p.capacity == 3 and p.available == 3
    a, b, c = p.acquire(), p.acquire(), p.acquire()
    with pytest.raises(MemoryError):
        p.acquire()
    mm.view(a, 64)[:] = 9
    p.release(a)
    with pytest.raises(ValueError):
        p.release(a)
    a2 = p.acquire()
    assert a2 == a and int(mm.view(a2, 64).sum()) == 0
    with pytest.raises(ValueError):
        p.release(1234)
    del b, c


def test_tiered_memory_fallthrough_and_migration():
    t = mm.TieredMemory([1000, 4000], names=["pinned", "pageable"])
    a = t.alloc(800, 0)
    b = t.alloc(800, 0)  # tier 0 is full: falls to tier 1
    assert t.tier_of(a) == 0 and t.tier_of(b) == 1 and t.name(1) == "pageable"
    assert not t.migrate(b, 0)  # no room
    assert t.migrate(a, 1) and t.used(0) == 0 and t.used(1) == 1600
    assert t.migrate(b, 0) and t.tier_of(b) == 0
    with pytest.raises(MemoryError):
        t.alloc(5000, 0)
    t.free(a)
    assert t.used(1) == 0
    with pytest.raises(ValueError):
        t.free(a)


@pytest.mark.parametrize("codec,bits", [("bfp8", 6), ("bfp4", 2)])
def test_block_floating_point_error_bound(codec, bits):
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(1000) * np.exp(rng.uniform(-6, 6, 1000))).astype(np.float32)
    x[100:132] = 0
    s = mm.compress(x, codec, block=32)
    y = mm.decompress(s, x.size)
    assert len(s) < (1.4 if codec == "bfp8" else 0.8) * x.size + 16
    for b0 in range(0, x.size, 32):
        blk = x[b0:b0 + 32]
        m = np.abs(blk).max()
        if m == 0:
            assert np.all(y[b0:b0 + 32] == 0)
            continue
        step = 2.0 ** (np.floor(np.log2(m)) - bits)
        # half a step of rounding, one step where the block maximum saturates the mantissa
        assert np.abs(y[b0:b0 + 32] - blk).max() <= step * 1.0001


def test_none_and_sparse_codecs():
    x = np.array([0.0, 3.0, -0.01, 0.5, -7.0, 0.02], dtype=np.float32)
    assert np.array_equal(mm.decompress(mm.compress(x, "none"), 6), x)
    y = mm.decompress(mm.compress(x, "sparse", threshold=0.1), 6)
    assert np.array_equal(y, np.array([0, 3.0, 0, 0.5, -7.0, 0], dtype=np.float32))
    with pytest.raises(KeyError):
        mm.compress(x, "zstd")
    with pytest.raises(ValueError):
        mm.decompress(b"short", 6)

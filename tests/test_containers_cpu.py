"""Host containers against Python's own dict / heapq / sorted lists under random operation sequences."""
import heapq
import random

from sneppx_alg_b200.utils.containers import HashTable, PriorityQueue, RBTree, strlcpy, strsplit


def test_hash_table_matches_dict():
    rng = random.Random(0)
    ht, ref = HashTable(8), {}
    for _ in range(20000):
        k = rng.randrange(3000) * 0x9E3779B97F4A7C15 % (1 << 64)
        op = rng.random()
        if op < 0.55:
            v = rng.getrandbits(63)
            ht[k] = v
            ref[k] = v
        elif op < 0.85:
            assert ht.get(k) == ref.get(k)
        else:
            if k in ref:
                del ht[k]
                del ref[k]
            else:
                assert k not in ht
    assert len(ht) == len(ref) and dict(ht.items()) == ref
    assert ht.capacity >= len(ref) / 0.7 - 1 and ht.max_probe < 40
    assert not ht.resize(8) and ht.resize(1 << 14) and dict(ht.items()) == ref
    ht.clear()
    assert len(ht) == 0 and ht.get(1) is None


def test_priority_queue_is_stable_min_heap():
    rng = random.Random(1)
    pq, ref, seq = PriorityQueue(), [], 0
    for _ in range(5000):
        if rng.random() < 0.6 or not ref:
            p, v = rng.randrange(50), rng.getrandbits(32)
            pq.push(p, v)
            heapq.heappush(ref, (p, seq, v))
            seq += 1
        else:
            p, _, v = heapq.heappop(ref)
            assert pq.peek() == (p, v) and pq.pop() == (p, v)
    assert len(pq) == len(ref)
    while ref:
        p, _, v = heapq.heappop(ref)
        assert pq.pop() == (p, v)
    assert pq.pop() is None


def test_red_black_tree_order_queries_and_balance():
    rng = random.Random(2)
    t, ref = RBTree(), {}
    for step in range(6000):
        k = rng.randrange(2000)
        if rng.random() < 0.6:
            assert t.insert(k, k * 3) == (k not in ref)
            ref[k] = k * 3
        else:
            assert t.delete(k) == (k in ref)
            ref.pop(k, None)
        if step % 500 == 0:
            assert t.black_height() >= 1
    keys = sorted(ref)
    assert [k for k, _ in t.items()] == keys and len(t) == len(keys) and t.black_height() >= 1
    assert t.min() == keys[0] and t.max() == keys[-1] and t.search(keys[5]) == keys[5] * 3
    for probe in (0, keys[3], keys[3] + 1, keys[-1], 5000):
        want_s = next((k for k in keys if k > probe), None)
        want_p = next((k for k in reversed(keys) if k < probe), None)
        assert t.successor(probe) == want_s and t.predecessor(probe) == want_p
    import math
    assert t.black_height() <= 2 * math.log2(len(keys) + 1)


def test_string_helpers():
    assert strlcpy("hello world", 6) == ("hello", 11)
    assert strsplit("a,b,,c", ",") == ["a", "b", "", "c"]
    assert strsplit("a,b,c,d", ",", max_tokens=2) == ["a", "b,c,d"]
    assert strsplit("single", ",") == ["single"]

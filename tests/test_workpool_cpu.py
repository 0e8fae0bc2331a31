"""Native work-stealing pool: futures, task groups (with helping waits), workloads, parallel_for / parallel_reduce,
and evidence that idle workers steal."""
import threading
import time

import pytest

from sneppx_alg_b200.utils.workpool import WorkStealingPool, Workload


def test_futures_results_and_exceptions():
    with WorkStealingPool(4) as pool:
        futs = [pool.submit(lambda x: x * x, i) for i in range(50)]
        assert [f.result(5) for f in futs] == [i * i for i in range(50)]
        bad = pool.submit(lambda: 1 / 0)
        with pytest.raises(ZeroDivisionError):
            bad.result(5)
        slow = pool.submit(time.sleep, 0.3)
        assert not slow.wait(0.01)
        with pytest.raises(TimeoutError):
            slow.result(0.01)
        assert slow.result(5) is None and slow.done()
        assert pool.map(lambda x: x + 1, range(10)) == list(range(1, 11))


def test_task_group_waits_and_nested_groups_do_not_deadlock():
    with WorkStealingPool(2) as pool:
        hits, lock = [], threading.Lock()

        def leaf(i):
            with lock:
                hits.append(i)

        def parent(base):
            # a task that spawns its own group and waits for it from inside the pool: the wait runs queued tasks
            g = pool.group()
            for j in range(8):
                g.add(leaf, base + j)
            assert g.wait(10)

        top = pool.group()
        for b in range(0, 64, 8):
            top.add(parent, b)
        assert top.wait(20)
        assert sorted(hits) == list(range(64)) and top.completed == 8
        g = pool.group()
        g.add(lambda: (_ for _ in ()).throw(ValueError("boom")))
        with pytest.raises(ValueError):
            g.wait(5)


def test_parallel_for_covers_range_once_and_work_is_stolen():
    with WorkStealingPool(4) as pool:
        n = 10_000
        seen = [0] * n

        def body(lo, hi):
            for i in range(lo, hi):
                seen[i] += 1
            time.sleep(0.0005)       # leaves time for other workers to steal the pushed halves
        pool.parallel_for(0, n, body, grain=100)
        assert seen == [1] * n
        assert pool.stats()["steals"] > 0
        total = pool.parallel_reduce(0, 1000, 0, lambda a, b, acc: acc + sum(range(a, b)), lambda x, y: x + y)
        assert total == sum(range(1000))
        # index-ordered combine: string concatenation is not commutative
        s = pool.parallel_reduce(0, 26, "", lambda a, b, acc: acc + "".join(chr(97 + i) for i in range(a, b)),
                                 lambda x, y: x + y)
        assert s == "abcdefghijklmnopqrstuvwxyz"


def test_workload_progress_timeout_and_cancel():
    with WorkStealingPool(2) as pool:
        wl = Workload(max_tasks=4)
        gate = threading.Event()
        done = []
        for i in range(4):
            assert wl.add_task(f"t{i}", lambda i=i: (gate.wait(5), done.append(i))) == i
        with pytest.raises(RuntimeError):
            wl.add_task("extra", lambda: None)
        assert wl.task_name(2) == "t2"
        wl.submit(pool)
        assert wl.wait(0.05) is False and wl.num_completed() == 0
        gate.set()
        assert wl.wait(10) and wl.num_completed() == 4 and sorted(done) == [0, 1, 2, 3]
        wl.close()
        # cancel: tasks not yet started are skipped
        wl2 = Workload()
        ran = []
        hold = threading.Event()
        wl2.add_task("first", lambda: hold.wait(5))
        for i in range(20):
            wl2.add_task(f"n{i}", lambda i=i: ran.append(i))
        wl2.submit(None, num_threads=1)
        time.sleep(0.05)
        wl2.cancel()
        hold.set()
        assert wl2.wait(10)
        assert len(ran) < 20 and wl2.num_completed() == 21
        wl2.close()

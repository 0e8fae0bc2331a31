"""Python face of the native work-stealing pool (``csrc/host/workpool.cpp``): futures, task groups, named
workloads, ``parallel_for`` / ``parallel_reduce``.

The pool's threads are C++ threads; a Python callable submitted to it runs under the interpreter lock like any other
Python code, so the gain is for callables that release it (NumPy / PyTorch kernels, I/O, ctypes calls into the host
library). The reference exposes the same shapes from C (futures and ``threadpool_submit_future``:
include/neural_core/kernel/concurrent_workload_dispatch.h:46-141; workloads and task groups:
kernel/thread/workload_dispatch.c:36-160) and binds ``_ThreadPool`` into Python.
"""
from __future__ import annotations

import ctypes as C
import threading
from typing import Callable, Iterable, List, Optional

from .. import _build

_TASK = C.CFUNCTYPE(None, C.c_void_p)
_RANGE = C.CFUNCTYPE(None, C.c_longlong, C.c_longlong, C.c_void_p)


def _L():
    L = _build.load_host()
    if not getattr(L, "_wp_ready", False):
        for f in ("sx_wp_create", "sx_wp_future_create", "sx_wp_group_create", "sx_wp_workload_create",
                  "sx_wp_future_get_result"):
            getattr(L, f).restype = C.c_void_p
        L.sx_wp_create.argtypes = [C.c_int]
        for f in ("sx_wp_destroy", "sx_wp_wait", "sx_wp_future_destroy", "sx_wp_group_destroy", "sx_wp_group_cancel",
                  "sx_wp_workload_destroy"):
            getattr(L, f).argtypes = [C.c_void_p]
            getattr(L, f).restype = None
        L.sx_wp_num_threads.argtypes = [C.c_void_p]
        L.sx_wp_stats.argtypes = [C.c_void_p, C.c_void_p]
        L.sx_wp_submit.argtypes = [C.c_void_p, _TASK, C.c_void_p]
        L.sx_wp_future_wait.argtypes = [C.c_void_p, C.c_int]
        L.sx_wp_future_is_ready.argtypes = [C.c_void_p]
        L.sx_wp_future_set_result.argtypes = [C.c_void_p, C.c_void_p]
        L.sx_wp_future_set_result.restype = None
        L.sx_wp_group_add.argtypes = [C.c_void_p, C.c_void_p, _TASK, C.c_void_p]
        L.sx_wp_group_wait.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.sx_wp_group_completed.argtypes = [C.c_void_p]
        L.sx_wp_group_completed.restype = C.c_longlong
        L.sx_wp_parallel_for.argtypes = [C.c_void_p, C.c_longlong, C.c_longlong, C.c_longlong, _RANGE, C.c_void_p]
        L.sx_wp_parallel_for.restype = None
        L.sx_wp_workload_create.argtypes = [C.c_longlong]
        L.sx_wp_workload_add_task.argtypes = [C.c_void_p, C.c_char_p, _TASK, C.c_void_p]
        L.sx_wp_workload_submit.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.sx_wp_workload_wait.argtypes = [C.c_void_p, C.c_int]
        L.sx_wp_workload_num_completed.argtypes = [C.c_void_p]
        L.sx_wp_workload_num_completed.restype = C.c_longlong
        L.sx_wp_workload_cancel.argtypes = [C.c_void_p]
        L.sx_wp_workload_task_name.argtypes = [C.c_void_p, C.c_int]
        L.sx_wp_workload_task_name.restype = C.c_char_p
        L._wp_ready = True
    return L


class Future:
    """Result slot of a submitted call: ``result(timeout)`` returns the value or re-raises the call's exception."""

    def __init__(self):
        self._h = _L().sx_wp_future_create()
        self._value, self._error, self._keep = None, None, None

    def done(self) -> bool:
        return bool(_L().sx_wp_future_is_ready(self._h))

    def wait(self, timeout: Optional[float] = None) -> bool:
        return bool(_L().sx_wp_future_wait(self._h, -1 if timeout is None else int(timeout * 1000)))

    def result(self, timeout: Optional[float] = None):
        if not self.wait(timeout):
            raise TimeoutError("future not ready")
        if self._error is not None:
            raise self._error
        return self._value

    def __del__(self):
        try:
            if self.done() or self._keep is None:
                _L().sx_wp_future_destroy(self._h)
        except Exception:  # noqa: BLE001  (interpreter shutdown)
            pass


class TaskGroup:
    """Tasks that are waited for together; ``wait`` helps running queued tasks instead of blocking."""

    def __init__(self, pool: "WorkStealingPool"):
        self.pool, self._h = pool, _L().sx_wp_group_create()
        self._keep: List = []
        self.errors: List[BaseException] = []

    def add(self, fn: Callable, *args, **kw) -> None:
        def run(_):
            try:
                fn(*args, **kw)
            except BaseException as e:  # noqa: BLE001  (reported by wait)
                self.errors.append(e)
        cb = _TASK(run)
        self._keep.append(cb)
        if _L().sx_wp_group_add(self.pool._h, self._h, cb, None) != 0:
            raise RuntimeError("task group rejected the task")

    def wait(self, timeout: Optional[float] = None) -> bool:
        ok = bool(_L().sx_wp_group_wait(self.pool._h, self._h, -1 if timeout is None else int(timeout * 1000)))
        if ok:
            self._keep.clear()
            if self.errors:
                raise self.errors[0]
        return ok

    def cancel(self) -> None:
        _L().sx_wp_group_cancel(self._h)

    @property
    def completed(self) -> int:
        return int(_L().sx_wp_group_completed(self._h))

    def __del__(self):
        try:
            if not self._keep:
                _L().sx_wp_group_destroy(self._h)
        except Exception:  # noqa: BLE001
            pass


class Workload:
    """A named list of tasks with progress and cancellation (``add_task`` / ``submit`` / ``wait`` /
    ``num_completed`` / ``cancel``)."""

    def __init__(self, max_tasks: int = 0):
        self._h = _L().sx_wp_workload_create(max_tasks)
        self._keep: List = []
        self.errors: List[BaseException] = []

    def add_task(self, name: str, fn: Callable, *args) -> int:
        def run(_):
            try:
                fn(*args)
            except BaseException as e:  # noqa: BLE001
                self.errors.append(e)
        cb = _TASK(run)
        i = _L().sx_wp_workload_add_task(self._h, name.encode(), cb, None)
        if i < 0:
            raise RuntimeError("workload is full")
        self._keep.append(cb)
        return i

    def task_name(self, i: int) -> str:
        return _L().sx_wp_workload_task_name(self._h, i).decode()

    def submit(self, pool: Optional["WorkStealingPool"] = None, num_threads: int = 2) -> None:
        if _L().sx_wp_workload_submit(self._h, pool._h if pool else None, num_threads) != 0:
            raise RuntimeError("workload was already submitted")

    def wait(self, timeout: Optional[float] = None) -> bool:
        return _L().sx_wp_workload_wait(self._h, -1 if timeout is None else int(timeout * 1000)) == 1

    def num_completed(self) -> int:
        return int(_L().sx_wp_workload_num_completed(self._h))

    def cancel(self) -> None:
        _L().sx_wp_workload_cancel(self._h)

    def close(self) -> None:
        if self._h:
            _L().sx_wp_workload_destroy(self._h)
            self._h = None


class WorkStealingPool:
    def __init__(self, workers: int = 0):
        self._h = _L().sx_wp_create(workers)
        self._lock = threading.Lock()
        self._live = {}

    @property
    def num_threads(self) -> int:
        return int(_L().sx_wp_num_threads(self._h))

    def stats(self) -> dict:
        out = (C.c_longlong * 3)()
        _L().sx_wp_stats(self._h, out)
        return {"executed": int(out[0]), "steals": int(out[1]), "queued": int(out[2])}

    def submit(self, fn: Callable, *args, **kw) -> Future:
        fut = Future()

        def run(_):
            try:
                fut._value = fn(*args, **kw)
            except BaseException as e:  # noqa: BLE001  (re-raised by Future.result)
                fut._error = e
            with self._lock:
                self._live.pop(id(fut), None)
            _L().sx_wp_future_set_result(fut._h, None)
        cb = _TASK(run)
        fut._keep = cb
        with self._lock:
            self._live[id(fut)] = (fut, cb)
        if _L().sx_wp_submit(self._h, cb, None) != 0:
            raise RuntimeError("pool rejected the task")
        return fut

    def map(self, fn: Callable, items: Iterable) -> list:
        futs = [self.submit(fn, x) for x in items]
        return [f.result() for f in futs]

    def group(self) -> TaskGroup:
        return TaskGroup(self)

    def parallel_for(self, start: int, end: int, body: Callable[[int, int], None], grain: int = 0) -> None:
        """Calls ``body(lo, hi)`` over disjoint chunks of [start, end); ranges are split in halves and idle workers
        steal the halves."""
        errors: List[BaseException] = []

        def run(lo, hi, _):
            try:
                body(int(lo), int(hi))
            except BaseException as e:  # noqa: BLE001
                errors.append(e)
        _L().sx_wp_parallel_for(self._h, start, end, grain, _RANGE(run), None)
        if errors:
            raise errors[0]

    def parallel_reduce(self, start: int, end: int, init, reduce_fn: Callable, combine_fn: Callable, grain: int = 0):
        """``reduce_fn(lo, hi, acc) -> acc`` over chunks, partial results merged with ``combine_fn(a, b)`` in index
        order (deterministic for non-commutative combines)."""
        if end <= start:
            return init
        parts = min(end - start, self.num_threads * 4) if grain <= 0 else max(1, (end - start + grain - 1) // grain)
        step = (end - start + parts - 1) // parts
        slots = [None] * parts

        def body(lo, hi):
            for i in range(lo, hi):
                a = start + i * step
                b = min(end, a + step)
                slots[i] = reduce_fn(a, b, init) if b > a else init
        self.parallel_for(0, parts, body, grain=1)
        acc = init
        for s in slots:
            acc = combine_fn(acc, s)
        return acc

    def wait(self) -> None:
        _L().sx_wp_wait(self._h)

    def shutdown(self) -> None:
        if self._h:
            self.wait()
            _L().sx_wp_destroy(self._h)
            self._h = None

    close = shutdown

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.shutdown()

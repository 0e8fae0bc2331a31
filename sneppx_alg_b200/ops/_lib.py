"""ctypes view of the CUDA kernel library (``csrc/sx_api.h``).

The library is loaded lazily on the first CUDA call. On a machine with a GPU a missing or
unloadable library is an error: there is no silent fallback to PyTorch kernels for CUDA tensors.
"""
from __future__ import annotations

import ctypes as C
import threading

import torch

from .. import _build

c_void_p, c_int, c_ll, c_float = C.c_void_p, C.c_int, C.c_longlong, C.c_float


class SxGemmArgs(C.Structure):
    _fields_ = [
        ("A", c_void_p), ("B", c_void_p), ("D", c_void_p), ("C", c_void_p), ("bias", c_void_p),
        ("M", c_int), ("N", c_int), ("K", c_int), ("batch", c_int),
        ("lda", c_ll), ("ldb", c_ll), ("ldd", c_ll), ("ldc", c_ll),
        ("strideA", c_ll), ("strideB", c_ll), ("strideD", c_ll), ("strideC", c_ll),
        ("a_mn", c_int), ("b_mn", c_int), ("out_fp32", c_int), ("c_fp32", c_int), ("act", c_int),
        ("alpha", c_float), ("beta", c_float),
        ("tile_group", c_void_p), ("num_groups", c_int),
        ("k_ranges", c_void_p), ("k_total", c_int),
        ("status", c_void_p), ("sm_limit", c_int), ("force_bn", c_int), ("flags", c_int),
    ]


class SxAttnArgs(C.Structure):
    _fields_ = [
        ("Q", c_void_p), ("K", c_void_p), ("V", c_void_p), ("O", c_void_p), ("lse", c_void_p),
        ("dO", c_void_p), ("dQ", c_void_p), ("dK", c_void_p), ("dV", c_void_p),
        ("dq_accum", c_void_p), ("delta", c_void_p),
        ("q_row_stride", c_ll), ("k_row_stride", c_ll), ("v_row_stride", c_ll), ("o_row_stride", c_ll),
        ("q_batch_stride", c_ll), ("k_batch_stride", c_ll), ("v_batch_stride", c_ll),
        ("do_row_stride", c_ll), ("dq_row_stride", c_ll), ("dk_row_stride", c_ll), ("dv_row_stride", c_ll),
        ("dq_batch_stride", c_ll), ("dk_batch_stride", c_ll), ("dv_batch_stride", c_ll),
        ("B", c_int), ("Sq", c_int), ("Skv", c_int), ("Hq", c_int), ("Hk", c_int), ("D", c_int),
        ("v_head_div", c_int), ("causal", c_int), ("window", c_int), ("scale", c_float),
        ("status", c_void_p),
        ("block_mask", c_void_p), ("bm_batch_stride", c_ll), ("bm_head_stride", c_ll),
    ]


_lock = threading.Lock()
_lib = None
_status = {}
launch_count = 0  # number of kernel-library entry points called (bench.py reports it)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                _lib = _build.load_cuda()
    return _lib


def available() -> bool:
    """True when CUDA tensors can be served by the native library."""
    if not torch.cuda.is_available():
        return False
    lib()  # raises if the library cannot be built / loaded: no silent fallback on a GPU box
    return True


def stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t) -> c_void_p:
    return c_void_p(0) if t is None else c_void_p(t.data_ptr())


def status_word(device=None) -> torch.Tensor:
    """Per-device int32 word the waiting kernels write their timeout codes into."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _status.get(key)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", key))
        _status[key] = t
    return t


STATUS_NAMES = {1: "TMA producer wait timed out", 2: "MMA issuer wait timed out", 3: "epilogue wait timed out",
                4: "peer signal wait timed out", 5: "bad argument", 6: "converter wait timed out"}


class KernelTimeout(RuntimeError):
    """A bounded device-side wait gave up; the CUDA context is still usable."""


def check_status(device=None, reset: bool = True) -> None:
    """Synchronising check of the device status word; raises KernelTimeout when a wait gave up."""
    t = status_word(device)
    code = int(t[0].item())
    if code != 0:
        if reset:
            t.zero_()
        raise KernelTimeout(f"sneppx kernel status {code}: {STATUS_NAMES.get(code, 'unknown')}")


class StatusPoll:
    """Non-blocking check of the status word: ``arm(stream)`` queues a 4-byte copy of the word into pinned host
    memory behind whatever the stream holds; ``check()`` raises KernelTimeout if an armed copy that has completed
    shows a code. A step calls ``check()`` on entry (reads the previous step's copy, which has landed by then)
    and ``arm()`` after its last launch, so a wait that ran out surfaces one step later without any
    host-device synchronisation on the hot path."""

    def __init__(self, device=None):
        self.word = status_word(device)
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.event = None

    def arm(self, stream=None):
        st = stream if stream is not None else torch.cuda.current_stream(self.word.device)
        with torch.cuda.stream(st):
            self.host.copy_(self.word[0:1], non_blocking=True)
            self.event = torch.cuda.Event()
            self.event.record(st)

    def check(self, wait: bool = False):
        if self.event is None:
            return
        if wait:
            self.event.synchronize()
        elif not self.event.query():
            return
        self.event = None
        code = int(self.host[0])
        if code != 0:
            self.word.zero_()
            raise KernelTimeout(f"sneppx kernel status {code}: {STATUS_NAMES.get(code, 'unknown')}")


def call(name: str, *args) -> None:
    global launch_count
    fn = getattr(lib(), name)
    rc = fn(*args)
    launch_count += 1
    if rc != 0:
        raise RuntimeError(f"{name} failed with code {rc}")

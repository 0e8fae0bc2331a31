"""The single device layer (the reference's ``drivers/cuda/cuda_driver.c:70-587`` and Python ``cuda_device.py`` /
``hw_backends.py``): device query, streams, events, pinned buffers, peer access — for CUDA sm_100a only; there is no
back-end dispatch."""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class DeviceProperties:
    name: str
    sm_count: int
    total_memory: int
    capability: tuple
    l2_bytes: int
    shared_per_block_optin: int

    @property
    def is_blackwell(self):
        return self.capability[0] == 10


def is_available() -> bool:
    return torch.cuda.is_available()


def device_count() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def properties(index: int = 0) -> DeviceProperties:
    p = torch.cuda.get_device_properties(index)
    return DeviceProperties(p.name, p.multi_processor_count, p.total_memory, (p.major, p.minor),
                            getattr(p, "L2_cache_size", 0), getattr(p, "shared_memory_per_block_optin", 0))


def require_b200(index: int = 0):
    """Raises unless the device is compute capability 10.x: the kernels are built for sm_100a only."""
    p = properties(index)
    if not p.is_blackwell:
        raise RuntimeError(f"{p.name} is compute capability {p.capability}; this package targets sm_100a")
    return p


def set_device(index: int):
    torch.cuda.set_device(index)


def synchronize(index=None):
    torch.cuda.synchronize(index)


Stream = torch.cuda.Stream
Event = torch.cuda.Event
current_stream = torch.cuda.current_stream
stream = torch.cuda.stream


def pinned_empty(*shape, dtype=torch.float32):
    return torch.empty(*shape, dtype=dtype, pin_memory=torch.cuda.is_available())


def memory_info(index: int = 0) -> dict:
    free, total = torch.cuda.mem_get_info(index)
    return {"free": free, "total": total, "allocated": torch.cuda.memory_allocated(index),
            "reserved": torch.cuda.memory_reserved(index)}


def can_access_peer(a: int, b: int) -> bool:
    return torch.cuda.can_device_access_peer(a, b)


def elapsed_ms(fn, iters=10, warmup=3) -> float:
    """CUDA-event timing on the current stream (the reference's ``SNEPPX_PROFILE_KERNEL`` macro)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = Event(enable_timing=True), Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters

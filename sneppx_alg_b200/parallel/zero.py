"""ZeRO-1/2/3 data-parallel engine over flat buffers (see ``ZeroEngine``); ``make_engine`` picks the
single-process engine when there is one rank."""
from __future__ import annotations

import torch.distributed as dist

from ..training.engine import TrainEngine


def make_engine(model, zero_stage=3, **kw):
    world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    if world == 1:
        return TrainEngine(model, **kw)
    from .zero_engine import ZeroEngine
    return ZeroEngine(model, zero_stage=zero_stage, **kw)

"""Data pipeline: in-memory / memory-mapped / streaming token datasets, batching ``DataLoader`` with a prefetch
thread and pinned staging, and the rank-strided ``DistributedSampler`` (``indices[rank::world]`` after an
epoch-seeded shuffle; interface_bindings/distributed.py:114-137, data_loader.py:99, kernel/data/data_pipeline.c)."""
from __future__ import annotations

import queue
import threading
from typing import Iterator, List

import numpy as np
import torch


class TensorDataset:
    def __init__(self, *tensors):
        assert all(len(t) == len(tensors[0]) for t in tensors)
        self.tensors = tensors

    def __len__(self):
        return len(self.tensors[0])

    def __getitem__(self, i):
        return tuple(t[i] for t in self.tensors)


class SyntheticTokenDataset:
    """Uniform random token ids of a fixed shape (the benchmark workloads)."""

    def __init__(self, vocab_size, seq_len, length=1 << 30, seed=0):
        self.vocab_size, self.seq_len, self.length, self.seed = vocab_size, seq_len, length, seed

    def __len__(self):
        return self.length

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + i)
        ids = torch.randint(0, self.vocab_size, (self.seq_len,), generator=g)
        return ids, ids


class MemoryMappedTextDataset:
    """Flat binary file of token ids (uint16 / int32) cut into fixed-length windows."""

    def __init__(self, path, seq_len, dtype=np.uint16, stride=None):
        self.data = np.memmap(path, dtype=dtype, mode="r")
        self.seq_len, self.stride = seq_len, stride or seq_len

    def __len__(self):
        return max(0, (len(self.data) - self.seq_len - 1) // self.stride + 1)

    def __getitem__(self, i):
        s = i * self.stride
        chunk = torch.from_numpy(self.data[s: s + self.seq_len + 1].astype(np.int64))
        return chunk[:-1], chunk[1:]


class StreamingTokenDataset:
    """Iterates an iterator of token lists, packing them into fixed-length samples."""

    def __init__(self, token_iter, seq_len, eos_id=0):
        self.it, self.seq_len, self.eos = token_iter, seq_len, eos_id

    def __iter__(self):
        buf: List[int] = []
        for toks in self.it:
            buf.extend(list(toks) + [self.eos])
            while len(buf) > self.seq_len:
                chunk = torch.tensor(buf[: self.seq_len + 1])
                buf = buf[self.seq_len:]
                yield chunk[:-1], chunk[1:]


class DistributedSampler:
    def __init__(self, dataset_len, num_replicas=1, rank=0, shuffle=True, seed=0, drop_last=False):
        self.n, self.world, self.rank, self.shuffle, self.seed, self.drop_last = dataset_len, num_replicas, rank, shuffle, seed, drop_last
        self.epoch = 0

    def set_epoch(self, epoch):
        self.epoch = epoch

    def indices(self) -> List[int]:
        idx = list(range(self.n))
        if self.shuffle:
            rng = np.random.RandomState(self.seed + self.epoch)
            rng.shuffle(idx)
        if self.drop_last:
            idx = idx[: len(idx) - len(idx) % self.world]
        return idx[self.rank:: self.world]

    def __iter__(self):
        return iter(self.indices())

    def __len__(self):
        return len(self.indices())


def default_collate(items):
    if isinstance(items[0], (tuple, list)):
        return tuple(default_collate([it[k] for it in items]) for k in range(len(items[0])))
    return torch.stack([torch.as_tensor(x) for x in items])


class DataLoader:
    def __init__(self, dataset, batch_size=1, shuffle=False, sampler=None, drop_last=True, prefetch=2, pin_memory=False,
                 collate_fn=default_collate, seed=0):
        self.ds, self.bs, self.drop_last, self.prefetch = dataset, batch_size, drop_last, prefetch
        self.pin = pin_memory and torch.cuda.is_available()
        self.collate = collate_fn
        self.sampler = sampler or (DistributedSampler(len(dataset), shuffle=shuffle, seed=seed) if hasattr(dataset, "__len__") else None)

    def _batches(self) -> Iterator:
        if self.sampler is None:
            items = []
            for it in self.ds:
                items.append(it)
                if len(items) == self.bs:
                    yield self.collate(items)
                    items = []
            if items and not self.drop_last:
                yield self.collate(items)
            return
        idx = list(self.sampler)
        for s in range(0, len(idx), self.bs):
            chunk = idx[s: s + self.bs]
            if len(chunk) < self.bs and self.drop_last:
                break
            yield self.collate([self.ds[i] for i in chunk])

    def __iter__(self):
        if self.prefetch <= 0:
            yield from self._batches()
            return
        q: queue.Queue = queue.Queue(maxsize=self.prefetch)
        stop = object()

        def worker():
            try:
                for b in self._batches():
                    if self.pin:
                        b = tuple(t.pin_memory() for t in b) if isinstance(b, tuple) else b.pin_memory()
                    q.put(b)
            finally:
                q.put(stop)
        threading.Thread(target=worker, daemon=True).start()
        while True:
            b = q.get()
            if b is stop:
                return
            yield b

    def __len__(self):
        n = len(self.sampler) if self.sampler is not None else 0
        return n // self.bs if self.drop_last else (n + self.bs - 1) // self.bs

"""Paged KV cache: a pool of fixed-size blocks with reference counts and copy-on-write forks, per-sequence block
tables and a prefix cache keyed by hashed token chunks. Same concepts as the reference's NumPy implementation
(interface_bindings/paged_attention.py:43-427: ``KVBlockPool``, ``PagedKVCache``, ``PrefixCache``), with the K/V
storage living on the GPU in the layout the decode kernel reads ([blocks, block_size, Hkv, D] per layer)."""
from __future__ import annotations

import hashlib
from collections import OrderedDict
from typing import Dict, List, Optional, Tuple

import torch


class KVBlockPool:
    """Block id allocator with refcounts (shared prefixes) and copy-on-write."""

    def __init__(self, num_blocks: int):
        self.num_blocks = num_blocks
        self.free: List[int] = list(range(num_blocks - 1, -1, -1))
        self.ref = [0] * num_blocks
        self.reclaim = None     # callable(n) -> blocks freed; set by the cache that owns prefix entries

    def allocate(self) -> int:
        if not self.free and self.reclaim is not None:
            self.reclaim(1)
        if not self.free:
            raise MemoryError("KV block pool exhausted")
        b = self.free.pop()
        self.ref[b] = 1
        return b

    def share(self, b: int) -> int:
        self.ref[b] += 1
        return b

    def release(self, b: int) -> None:
        self.ref[b] -= 1
        if self.ref[b] == 0:
            self.free.append(b)
        elif self.ref[b] < 0:
            raise RuntimeError(f"double free of KV block {b}")

    @property
    def num_free(self) -> int:
        return len(self.free)


class PrefixCache:
    """Maps a hash of (all tokens up to the end of a full block) to the block that holds their K/V. Entries are
    kept in least-recently-used order; the cache never pins more than ``max_entries`` blocks (by default half of
    the pool) and gives blocks back on demand (``evict``) when the pool runs short."""

    def __init__(self, pool: KVBlockPool, block_size: int, max_entries: Optional[int] = None):
        if max_entries is None:
            max_entries = max(1, min(4096, pool.num_blocks // 2))
        self.pool, self.block_size, self.max_entries = pool, block_size, max_entries
        self.table: "OrderedDict[bytes, int]" = OrderedDict()

    @staticmethod
    def _hash(prev: bytes, chunk) -> bytes:
        h = hashlib.blake2b(digest_size=16)
        h.update(prev)
        h.update(bytes(str(list(chunk)), "ascii"))
        return h.digest()

    def match(self, tokens) -> Tuple[List[int], List[bytes]]:
        """Longest cached run of full blocks; returns (block ids with a new reference each, their keys)."""
        blocks, keys, prev = [], [], b""
        for i in range(0, len(tokens) - len(tokens) % self.block_size, self.block_size):
            key = self._hash(prev, tokens[i: i + self.block_size])
            b = self.table.get(key)
            if b is None:
                break
            self.table.move_to_end(key)
            blocks.append(self.pool.share(b))
            keys.append(key)
            prev = key
        return blocks, keys

    def insert(self, tokens, block_ids) -> None:
        prev = b""
        for j, i in enumerate(range(0, len(tokens) - len(tokens) % self.block_size, self.block_size)):
            key = self._hash(prev, tokens[i: i + self.block_size])
            if key in self.table:
                self.table.move_to_end(key)
            elif j < len(block_ids):
                if len(self.table) >= self.max_entries:
                    _, old = self.table.popitem(last=False)
                    self.pool.release(old)
                self.table[key] = self.pool.share(block_ids[j])
            prev = key

    def evictable(self) -> int:
        """Blocks that only the cache still holds."""
        return sum(1 for b in self.table.values() if self.pool.ref[b] == 1)

    def evict(self, n: int) -> int:
        """Give back up to ``n`` blocks that no running sequence shares, least recently used first."""
        freed = 0
        for key in list(self.table):
            if freed >= n:
                break
            b = self.table[key]
            if self.pool.ref[b] == 1:
                del self.table[key]
                self.pool.release(b)
                freed += 1
        return freed


class PagedKVCache:
    def __init__(self, num_layers, num_blocks, block_size, num_kv_heads, head_dim, dtype=torch.bfloat16, device="cuda",
                 enable_prefix_cache=True):
        self.block_size, self.num_layers = block_size, num_layers
        self.pool = KVBlockPool(num_blocks)
        shape = (num_blocks, block_size, num_kv_heads, head_dim)
        self.k = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(num_layers)]
        self.v = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(num_layers)]
        self.tables: Dict[int, List[int]] = {}
        self.lens: Dict[int, int] = {}
        self.prefix = PrefixCache(self.pool, block_size) if enable_prefix_cache else None
        if self.prefix is not None:
            self.pool.reclaim = self.prefix.evict

    def available_blocks(self) -> int:
        """Free blocks plus those the prefix cache would give back."""
        return self.pool.num_free + (self.prefix.evictable() if self.prefix is not None else 0)

    def make_room(self, n: int) -> bool:
        """Evict prefix entries until ``n`` blocks are free; False if that is not possible."""
        short = n - self.pool.num_free
        if short > 0 and self.prefix is not None:
            self.prefix.evict(short)
        return self.pool.num_free >= n

    # ---- sequences
    def add_sequence(self, seq_id: int, tokens=None) -> int:
        """Registers a sequence; returns how many prompt tokens are already covered by cached prefix blocks."""
        blocks = []
        if self.prefix is not None and tokens is not None:
            blocks, _ = self.prefix.match(tokens)
            # always leave at least one token to compute so that the model produces logits
            while blocks and len(blocks) * self.block_size >= len(tokens):
                self.pool.release(blocks.pop())
        self.tables[seq_id] = blocks
        self.lens[seq_id] = len(blocks) * self.block_size
        return self.lens[seq_id]

    def reserve(self, seq_id: int, n_new: int) -> List[int]:
        """Slots (block * block_size + offset) for the next ``n_new`` tokens, allocating / copying blocks as needed."""
        table, n = self.tables[seq_id], self.lens[seq_id]
        slots = []
        for i in range(n, n + n_new):
            bi, off = divmod(i, self.block_size)
            if bi == len(table):
                table.append(self.pool.allocate())
            elif self.pool.ref[table[bi]] > 1:      # shared block about to be written: copy on write
                new = self.pool.allocate()
                for l in range(self.num_layers):
                    self.k[l][new].copy_(self.k[l][table[bi]])
                    self.v[l][new].copy_(self.v[l][table[bi]])
                self.pool.release(table[bi])
                table[bi] = new
            slots.append(table[bi] * self.block_size + off)
        self.lens[seq_id] = n + n_new
        return slots

    def fork(self, src_id: int, dst_id: int) -> None:
        self.tables[dst_id] = [self.pool.share(b) for b in self.tables[src_id]]
        self.lens[dst_id] = self.lens[src_id]

    def free_sequence(self, seq_id: int, tokens=None) -> None:
        table = self.tables.pop(seq_id, [])
        n = self.lens.pop(seq_id, 0)
        if self.prefix is not None and tokens is not None:
            self.prefix.insert(tokens[:n], table)
        for b in table:
            self.pool.release(b)

    def block_table_tensor(self, seq_ids, device=None) -> Tuple[torch.Tensor, torch.Tensor]:
        mb = max(1, max(len(self.tables[s]) for s in seq_ids))
        bt = torch.zeros(len(seq_ids), mb, dtype=torch.int32)
        for i, s in enumerate(seq_ids):
            t = self.tables[s]
            bt[i, : len(t)] = torch.tensor(t, dtype=torch.int32)
        lens = torch.tensor([self.lens[s] for s in seq_ids], dtype=torch.int32)
        dev = device or self.k[0].device
        return bt.to(dev), lens.to(dev)

    def gather(self, layer: int, seq_id: int, n: Optional[int] = None):
        """Contiguous [n, Hkv, D] K and V of a sequence (used when a prefill chunk attends to cached tokens)."""
        n = self.lens[seq_id] if n is None else n
        blocks = torch.tensor(self.tables[seq_id][: (n + self.block_size - 1) // self.block_size], dtype=torch.long,
                              device=self.k[layer].device)
        k = self.k[layer][blocks].reshape(-1, *self.k[layer].shape[2:])[:n]
        v = self.v[layer][blocks].reshape(-1, *self.v[layer].shape[2:])[:n]
        return k, v

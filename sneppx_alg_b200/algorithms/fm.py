"""FM — federated memory: per-node key/value memory banks, a controller, and synchronisation (weighted all-reduce,
gossip, ring topology) with top-k compression + error feedback, Laplace differential-privacy noise and an adaptive
sync interval (algorithms/fm/core/{memory_bank,node,controller,forward,sync}.c; CUDA twin fm_cuda.cu; Python
``algo_fm.py`` with ``FMSyncNCCL``).

Banks are dense device tensors and every bank operation is batched: a read scores all entries with one distance
computation; a controller-level sync averages all slots of all nodes in one reduction.  ``FMSyncNCCL`` averages banks
across ranks with one real all-reduce (the reference simulates the collective inside a single buffer)."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..nn.modules import Module

SYNC_ALL_REDUCE, SYNC_GOSSIP, SYNC_TOPOLOGY = 0, 1, 2


@dataclass
class FMConfig:
    """``SNEPPX_fm_config_default`` (controller.c:28-41)."""
    num_nodes: int = 4
    memory_dim: int = 512
    memory_capacity: int = 1024
    sync_interval: int = 100
    sync_method: int = SYNC_ALL_REDUCE
    compression_ratio: float = 0.1
    privacy_epsilon: float = 1.0
    catastrophic_forgetting_protection: bool = True
    ewm_alpha: float = 0.9


def similarity(keys, q):
    """1 / (1 + mean squared distance) (memory_bank.c:25-32); keys [n, d], q [d] or [m, d] -> [n] or [m, n]."""
    d2 = torch.cdist(q.reshape(-1, q.shape[-1]).float(), keys.float()).pow(2) / keys.shape[-1]
    s = 1.0 / (1.0 + d2)
    return s[0] if q.dim() == 1 else s


class MemoryBank:
    def __init__(self, dim, capacity, device=None):
        self.keys = torch.zeros(capacity, dim, device=device)
        self.values = torch.zeros(capacity, dim, device=device)
        self.timestamps = torch.zeros(capacity, device=device)
        self.access = torch.zeros(capacity, device=device)
        self.num_entries, self.capacity = 0, capacity

    def write(self, key, value):
        """Overwrite a near-duplicate (similarity > 0.95), else append, else evict the entry with the lowest
        access / age score (memory_bank.c:84-139)."""
        n = self.num_entries
        now = float(n)
        if n:
            sim = similarity(self.keys[:n], key)
            best = int(sim.argmax())
            if float(sim[best]) > 0.95:
                self.values[best] = value
                self.timestamps[best], self.access[best] = now, 0.0
                return best
        if n < self.capacity:
            idx = n
            self.num_entries += 1
        else:
            age = (now - self.timestamps).clamp_min(1.0)
            idx = int((self.access / age).argmin())
        self.keys[idx], self.values[idx] = key, value
        self.timestamps[idx], self.access[idx] = now, 0.0
        return idx

    def read(self, key):
        """Value of the most similar entry, or None below similarity 0.5 (memory_bank.c:141-176)."""
        n = self.num_entries
        if n == 0:
            return None
        sim = similarity(self.keys[:n], key)
        best = int(sim.argmax())
        if float(sim[best]) < 0.5:
            return None
        self.access[best] += 1.0
        self.timestamps[best] = float(n)
        return self.values[best].clone()

    def read_batch(self, keys, threshold=0.5):
        """Batched read without bookkeeping: (values [m, d], hit mask [m])."""
        n = self.num_entries
        if n == 0:
            return torch.zeros_like(keys), torch.zeros(keys.shape[0], dtype=torch.bool, device=keys.device)
        sim = similarity(self.keys[:n], keys)
        best_sim, best = sim.max(-1)
        return self.values[best], best_sim >= threshold

    def forget(self, rate):
        """Clears the ``rate`` fraction with the lowest access^2 / age retention score (memory_bank.c:191-226)."""
        n = self.num_entries
        k = min(int(rate * n), n - 1)
        if n == 0 or k <= 0:
            return 0
        age = (float(n) - self.timestamps[:n]).clamp_min(1.0)
        drop = torch.topk(self.access[:n] ** 2 / age, k, largest=False).indices
        for t in (self.keys, self.values):
            t[drop] = 0
        self.timestamps[drop] = 0
        self.access[drop] = 0
        return k


class ErrorFeedback:
    """Top-k compression with residual accumulation (sync.c:268-334)."""

    def __init__(self, ratio=0.1):
        self.ratio, self.residual = ratio, None

    def compress(self, grad):
        acc = grad if self.residual is None else grad + self.residual
        out = compress_topk(acc, self.ratio)
        self.residual = acc - out
        return out


def compress_topk(grad, ratio):
    """Keeps the ``ratio`` largest-magnitude entries, zeroes the rest (sync.c:69-118)."""
    if ratio >= 1.0:
        return grad.clone()
    flat = grad.reshape(-1)
    keep = max(1, min(flat.numel(), int(ratio * flat.numel())))
    idx = torch.topk(flat.abs(), keep).indices
    out = torch.zeros_like(flat)
    out[idx] = flat[idx]
    return out.view_as(grad)


def compress_block_top2(grad):
    """Keeps the two largest-magnitude entries of every 32 (fm_cuda.cu:176-209); returns (kept, residual). The block
    form needs no global sort, so it is one bandwidth-bound pass; the tail that does not fill a block is kept."""
    from ..ops import aux
    flat = grad.reshape(-1).float()
    n = flat.numel() // 32 * 32
    kept, res = aux.block_top2(flat[:n]) if n else (flat[:0], flat[:0])
    return torch.cat([kept, flat[n:]]).view_as(grad), torch.cat([res, torch.zeros_like(flat[n:])]).view_as(grad)


class BlockErrorFeedback:
    """Error feedback around ``compress_block_top2``: what a step drops is added to the next gradient."""

    def __init__(self):
        self.residual = None

    def compress(self, grad):
        acc = grad.float() if self.residual is None else grad.float() + self.residual
        kept, self.residual = compress_block_top2(acc)
        return kept


def quantize_grad_int8(grad):
    """int8 codes with one scale per 256 values (fm_cuda.cu:100-173); returns (codes, scales, numel). The buffer is
    zero-padded to a multiple of 256."""
    from ..ops import aux
    flat = grad.reshape(-1).float()
    pad = (-flat.numel()) % 256
    if pad:
        flat = torch.cat([flat, flat.new_zeros(pad)])
    q, s = aux.quant_int8(flat)
    return q, s, grad.numel()


def dequantize_grad_int8(q, scales, numel, shape=None):
    from ..ops import aux
    y = aux.dequant_int8(q, scales)[:numel]
    return y.view(shape) if shape is not None else y


def federated_average(tensors, weights=None):
    """Weighted mean of the nodes' buffers (fm_cuda.cu:225-240); weights default to uniform and are normalised."""
    from ..ops import aux
    w = [1.0] * len(tensors) if weights is None else [float(v) for v in weights]
    tot = sum(w)
    return aux.weighted_average(list(tensors), [v / tot for v in w]).view_as(tensors[0])


def add_privacy_noise(t, epsilon, generator=None):
    """In-place Laplace(0, 1/epsilon) noise (sync.c:41-47)."""
    if epsilon <= 0:
        return t
    u = torch.rand(t.shape, device=t.device, generator=generator) - 0.5
    return t.add_(-(1.0 / epsilon) * u.sign() * torch.log1p(-2 * u.abs()))


class Node:
    def __init__(self, node_id, dim, capacity, device=None):
        self.node_id, self.bank = node_id, MemoryBank(dim, capacity, device)
        self.is_online, self.trust_score, self.last_sync = True, 1.0, 0
        self.grad_acc = torch.zeros(dim, device=device)


class FMController(Module):
    def __init__(self, cfg: FMConfig = None, device=None, **kw):
        super().__init__()
        self.cfg = cfg or FMConfig(**kw)
        c = self.cfg
        self.nodes = [Node(i, c.memory_dim, c.memory_capacity, device) for i in range(c.num_nodes)]
        self.contributions = [0.0] * c.num_nodes
        self.step_counter, self.sync_round, self.conflicts = 0, 0, []
        self.error_feedback = [ErrorFeedback(c.compression_ratio) for _ in range(c.num_nodes)]

    # ---- forward (forward.c:33-94): blend with the retrieved memory, else store the input
    def forward(self, x, node_id=0):
        node = self.nodes[node_id]
        if not node.is_online:
            raise RuntimeError(f"node {node_id} is offline")
        flat = x.reshape(-1, x.shape[-1]).float()
        if flat.shape[0] == 1:
            got = node.bank.read(flat[0])
            if got is None:
                node.bank.write(flat[0], flat[0])
                out = flat
            else:
                out = (self.cfg.ewm_alpha * flat[0] + (1 - self.cfg.ewm_alpha) * got)[None]
        else:
            vals, hit = node.bank.read_batch(flat)
            out = torch.where(hit[:, None], self.cfg.ewm_alpha * flat + (1 - self.cfg.ewm_alpha) * vals, flat)
            miss = (~hit).nonzero().flatten()[:4]          # store a few unseen rows per call
            for i in miss.tolist():
                node.bank.write(flat[i].detach(), flat[i].detach())
        node.grad_acc += 0.01 * out.detach().mean(0)
        self.step_counter += 1
        if self.cfg.sync_interval > 0 and self.step_counter % self.cfg.sync_interval == 0:
            self.sync()
        return out.to(x.dtype).view_as(x)

    def sync(self):
        return {SYNC_ALL_REDUCE: self.sync_all_reduce, SYNC_GOSSIP: self.sync_gossip,
                SYNC_TOPOLOGY: self.sync_topology}[self.cfg.sync_method]()

    # ---- trust-weighted average of every slot over the online nodes (sync.c:141-217)
    def sync_all_reduce(self):
        on = [n for n in self.nodes if n.is_online]
        if not on:
            return 1
        slots = max(n.bank.num_entries for n in on)
        if slots:
            w = torch.stack([(torch.arange(slots, device=n.bank.keys.device) < n.bank.num_entries).float() * n.trust_score
                             for n in on])                                              # [nodes, slots]
            tot = w.sum(0).clamp_min(1e-10)[:, None]
            k = sum(n.bank.keys[:slots] * w[i][:, None] for i, n in enumerate(on)) / tot
            v = sum(n.bank.values[:slots] * w[i][:, None] for i, n in enumerate(on)) / tot
            var = sum(((n.bank.values[:slots] - v) ** 2 * (w[i] > 0)[:, None]).sum(-1) for i, n in enumerate(on)) / \
                (len(self.nodes) * self.cfg.memory_dim)
            self.conflicts.extend((var > 0.1).nonzero().flatten().tolist())
            for n in on:
                n.bank.keys[:slots], n.bank.values[:slots] = k, v
                n.bank.num_entries = max(n.bank.num_entries, slots)
        self.sync_round += 1
        for n in on:
            n.last_sync = self.step_counter
            self.contributions[n.node_id] += 0.1
        return 0

    def _average_pair(self, a, b, alpha=0.5):
        m = min(a.bank.num_entries, b.bank.num_entries)
        if m:
            for name in ("keys", "values"):
                ta, tb = getattr(a.bank, name), getattr(b.bank, name)
                avg = alpha * ta[:m] + (1 - alpha) * tb[:m]
                ta[:m], tb[:m] = avg, avg

    def sync_gossip(self, num_pairs=None, seed=None):
        """Random pairs of online nodes average their banks (sync.c:219-241)."""
        on = [n for n in self.nodes if n.is_online]
        g = torch.Generator().manual_seed(self.sync_round if seed is None else seed)
        for _ in range(num_pairs or len(self.nodes)):
            if len(on) < 2:
                break
            i, j = torch.randperm(len(on), generator=g)[:2].tolist()
            self._average_pair(on[i], on[j])
        self.sync_round += 1
        return 0

    def sync_topology(self):
        """Ring: every online node averages with its right neighbour (sync.c:243-266)."""
        on = [n for n in self.nodes if n.is_online]
        for i in range(len(on)):
            self._average_pair(on[i], on[(i + 1) % len(on)])
        self.sync_round += 1
        return 0

    def adaptive_sync_interval(self, base=100.0):
        """base / (1 + stddev of node contributions), clamped to [0.1, 2] x base (sync.c:389-424)."""
        c = torch.tensor([self.contributions[n.node_id] for n in self.nodes if n.is_online])
        if c.numel() == 0:
            return int(base)
        mult = float((1.0 / (1.0 + c.std(unbiased=False))).clamp(0.1, 2.0))
        return int(max(base, 1.0) * mult + 0.5)

    def change_rate(self, node_id, new_values):
        b = self.nodes[node_id].bank
        n = min(b.num_entries, new_values.shape[0])
        return float((new_values[:n] - b.values[:n]).abs().mean()) if n else 0.0

    def send_gradients(self, node_id, grad):
        """Compress with error feedback, add DP noise, accumulate at the node (sync.c:426-449)."""
        g = self.error_feedback[node_id].compress(grad.float())
        add_privacy_noise(g, self.cfg.privacy_epsilon * 1e3)
        self.nodes[node_id].grad_acc = g
        return g

    def receive_gradients(self):
        on = [n for n in self.nodes if n.is_online]
        return sum(n.grad_acc * n.trust_score for n in on) / max(1e-10, sum(n.trust_score for n in on))


class FMSyncNCCL:
    """Cross-rank bank averaging with one all-reduce per tensor (the reference's ``SNEPPX_fm_sync_nccl`` callback hook,
    sync.c:482-497). Works on any initialised process group (NCCL on GPUs, gloo on CPU)."""

    def __init__(self, controller: FMController, group=None):
        self.ctrl, self.group = controller, group

    def sync(self, node_id=0):
        b = self.ctrl.nodes[node_id].bank
        if not (dist.is_available() and dist.is_initialized()):
            return 0
        world = dist.get_world_size(self.group)
        n = torch.tensor([b.num_entries], device=b.keys.device)
        dist.all_reduce(n, op=dist.ReduceOp.MAX, group=self.group)
        m = int(n)
        for t in (b.keys, b.values):
            dist.all_reduce(t[:m], group=self.group)
            t[:m] /= world
        b.num_entries = max(b.num_entries, m)
        self.ctrl.sync_round += 1
        return 0


FMModel = FMController

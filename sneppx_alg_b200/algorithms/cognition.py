"""Cognitive memory: episodic (prioritised transition buffer), semantic (concept embeddings with relations and LRU
forgetting), working (attended slots) and procedural (state -> skill cache that compiles frequent skills) stores, and
the forward pass that concatenates what each store returns for an input.

Reference: ``kernel/memory/cognition/{episodic,semantic,working,procedural,cognitive_manager}.c`` and
``include/neural_core/architecture/cognitive_memory.h`` (``SNEPPX_cognitive_memory_forward`` at
``cognitive_manager.c:169-225``: output = [input | attended working slot | mean of the 3 nearest concepts | recalled
skill]). Stores are torch tensors on one device; similarity searches are single matmuls, so a store of thousands of
entries is one small GEMM instead of the reference's per-entry loops.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F


@dataclass
class EpisodicConfig:
    capacity: int = 1024
    max_priority_samples: int = 64
    consolidation_interval: int = 256


@dataclass
class SemanticConfig:
    max_concepts: int = 512
    max_edges: int = 2048
    embedding_dim: int = 64
    lru_size: int = 64


@dataclass
class WorkingConfig:
    num_slots: int = 8
    slot_dim: int = 64


@dataclass
class ProceduralConfig:
    cache_size: int = 128
    state_dim: int = 64
    skill_dim: int = 32
    compilation_threshold: int = 3


@dataclass
class CognitiveMemoryConfig:
    episodic: EpisodicConfig = field(default_factory=EpisodicConfig)
    semantic: SemanticConfig = field(default_factory=SemanticConfig)
    working: WorkingConfig = field(default_factory=WorkingConfig)
    procedural: ProceduralConfig = field(default_factory=ProceduralConfig)


def _fit(v: torch.Tensor, dim: int) -> torch.Tensor:
    """Flatten and truncate / zero-pad to `dim`."""
    v = v.reshape(-1).float()
    return v[:dim] if v.numel() >= dim else F.pad(v, (0, dim - v.numel()))


class EpisodicMemory:
    """Ring buffer of (state, action, reward, next_state) with priority = |reward| + eps."""

    def __init__(self, cfg: EpisodicConfig, device="cpu", seed: int = 0):
        self.cfg, self.device = cfg, device
        self.items: List[Tuple[torch.Tensor, torch.Tensor, float, torch.Tensor]] = []
        self.priority: List[float] = []
        self.head = 0
        self.recorded = 0
        self.gen = torch.Generator(device="cpu").manual_seed(seed)

    def record(self, state, action, reward: float, next_state) -> bool:
        """Returns True when this record reaches the consolidation interval."""
        item = (state.detach().to(self.device).reshape(-1).float(), action.detach().to(self.device).reshape(-1).float(),
                float(reward), next_state.detach().to(self.device).reshape(-1).float())
        if len(self.items) < self.cfg.capacity:
            self.items.append(item)
            self.priority.append(abs(reward) + 1e-3)
        else:
            self.items[self.head] = item
            self.priority[self.head] = abs(reward) + 1e-3
        self.head = (self.head + 1) % self.cfg.capacity
        self.recorded += 1
        return self.recorded % self.cfg.consolidation_interval == 0

    def retrieve(self, query, k: int = 1):
        """The k transitions whose state is nearest (cosine) to `query`: list of (index, similarity)."""
        if not self.items:
            return []
        S = torch.stack([_fit(s, query.numel()) for s, _, _, _ in self.items])
        sim = F.cosine_similarity(S, query.reshape(1, -1).float().to(self.device), dim=1)
        top = torch.topk(sim, min(k, len(self.items)))
        return [(int(i), float(v)) for v, i in zip(top.values, top.indices)]

    def sample(self, n: int) -> List[int]:
        """Priority-proportional sample without replacement (at most max_priority_samples)."""
        n = min(n, len(self.items), self.cfg.max_priority_samples)
        if n == 0:
            return []
        p = torch.tensor(self.priority)
        return torch.multinomial(p / p.sum(), n, replacement=False, generator=self.gen).tolist()

    def __len__(self):
        return len(self.items)


class SemanticMemory:
    """Concept id -> embedding, undirected weighted relations, least-recently-used forgetting at capacity."""

    def __init__(self, cfg: SemanticConfig, device="cpu"):
        self.cfg, self.device = cfg, device
        self.emb = torch.zeros(cfg.max_concepts, cfg.embedding_dim, device=device)
        self.ids: List[Optional[int]] = [None] * cfg.max_concepts
        self.slot: Dict[int, int] = {}
        self.clock = 0
        self.last_use = [0] * cfg.max_concepts
        self.edges: Dict[Tuple[int, int], float] = {}

    def store(self, concept_id: int, embedding) -> int:
        self.clock += 1
        if concept_id in self.slot:
            s = self.slot[concept_id]
        elif len(self.slot) < self.cfg.max_concepts:
            s = self.ids.index(None)
        else:  # evict the least recently used concept and its relations
            s = min(range(self.cfg.max_concepts), key=lambda i: self.last_use[i])
            self.forget(self.ids[s])
        self.ids[s], self.slot[concept_id], self.last_use[s] = concept_id, s, self.clock
        self.emb[s] = _fit(embedding.detach().to(self.device), self.cfg.embedding_dim)
        return s

    def retrieve(self, query, k: int = 3):
        """(embeddings [m, D], ids) of the m <= k concepts nearest to `query` by cosine similarity."""
        if not self.slot:
            return torch.zeros(0, self.cfg.embedding_dim, device=self.device), []
        live = torch.tensor(sorted(self.slot.values()), device=self.device)
        q = _fit(query.to(self.device), self.cfg.embedding_dim).unsqueeze(0)
        sim = F.cosine_similarity(self.emb[live], q, dim=1)
        top = torch.topk(sim, min(k, live.numel())).indices
        rows = live[top].tolist()
        self.clock += 1
        for r in rows:
            self.last_use[r] = self.clock
        return self.emb[rows], [self.ids[r] for r in rows]

    def relate(self, a: int, b: int, weight: float = 1.0) -> bool:
        if a not in self.slot or b not in self.slot or a == b:
            return False
        key = (min(a, b), max(a, b))
        if key not in self.edges and len(self.edges) >= self.cfg.max_edges:
            return False
        self.edges[key] = weight
        return True

    def neighbours(self, a: int) -> Dict[int, float]:
        return {(y if x == a else x): w for (x, y), w in self.edges.items() if a in (x, y)}

    def forget(self, concept_id: int) -> bool:
        s = self.slot.pop(concept_id, None)
        if s is None:
            return False
        self.ids[s] = None
        self.emb[s].zero_()
        self.edges = {k: w for k, w in self.edges.items() if concept_id not in k}
        return True


class WorkingMemory:
    """Fixed slots; `attend` reads a softmax(q . slot / sqrt(d))-weighted mixture of the written slots."""

    def __init__(self, cfg: WorkingConfig, device="cpu"):
        self.cfg = cfg
        self.slots = torch.zeros(cfg.num_slots, cfg.slot_dim, device=device)
        self.valid = torch.zeros(cfg.num_slots, dtype=torch.bool, device=device)

    def write(self, slot: int, value):
        if not 0 <= slot < self.cfg.num_slots:
            raise IndexError(slot)
        self.slots[slot] = _fit(value.detach().to(self.slots.device), self.cfg.slot_dim)
        self.valid[slot] = True

    def read(self, slot: int) -> Optional[torch.Tensor]:
        return self.slots[slot].clone() if bool(self.valid[slot]) else None

    def attend(self, query) -> torch.Tensor:
        if not bool(self.valid.any()):
            return torch.zeros(self.cfg.slot_dim, device=self.slots.device)
        q = _fit(query.to(self.slots.device), self.cfg.slot_dim)
        score = (self.slots @ q) / self.cfg.slot_dim ** 0.5
        w = torch.softmax(score.masked_fill(~self.valid, float("-inf")), dim=0)
        return w @ self.slots

    def clear(self):
        self.slots.zero_()
        self.valid.zero_()


class ProceduralMemory:
    """State -> skill pairs. A pair used `compilation_threshold` times is moved into the compiled matrix, which is
    searched first (one matmul) and exempt from eviction."""

    def __init__(self, cfg: ProceduralConfig, device="cpu"):
        self.cfg, self.device = cfg, device
        self.states: List[torch.Tensor] = []
        self.skills: List[torch.Tensor] = []
        self.uses: List[int] = []
        self.compiled_states = torch.zeros(0, cfg.state_dim, device=device)
        self.compiled_skills = torch.zeros(0, cfg.skill_dim, device=device)

    def learn(self, state, skill):
        if len(self.states) >= self.cfg.cache_size:  # drop the least used
            i = min(range(len(self.uses)), key=self.uses.__getitem__)
            for l in (self.states, self.skills, self.uses):
                l.pop(i)
        self.states.append(_fit(state.detach().to(self.device), self.cfg.state_dim))
        self.skills.append(_fit(skill.detach().to(self.device), self.cfg.skill_dim))
        self.uses.append(0)

    def recall(self, state, min_similarity: float = 0.0) -> Optional[torch.Tensor]:
        q = _fit(state.to(self.device), self.cfg.state_dim).unsqueeze(0)
        best, best_sim = None, min_similarity
        if self.compiled_states.shape[0]:
            sim = F.cosine_similarity(self.compiled_states, q, dim=1)
            v, i = sim.max(0)
            if float(v) > best_sim:
                best, best_sim = self.compiled_skills[int(i)], float(v)
        if self.states:
            sim = F.cosine_similarity(torch.stack(self.states), q, dim=1)
            v, i = sim.max(0)
            if float(v) > best_sim:
                best, best_sim = self.skills[int(i)], float(v)
                self.uses[int(i)] += 1
        return None if best is None else best.clone()

    def compile(self) -> int:
        """Moves every pair at or above the use threshold into the compiled matrix; returns how many moved."""
        hot = [i for i, u in enumerate(self.uses) if u >= self.cfg.compilation_threshold]
        if not hot:
            return 0
        self.compiled_states = torch.cat([self.compiled_states, torch.stack([self.states[i] for i in hot])])
        self.compiled_skills = torch.cat([self.compiled_skills, torch.stack([self.skills[i] for i in hot])])
        for i in reversed(hot):
            for l in (self.states, self.skills, self.uses):
                l.pop(i)
        return len(hot)


class CognitiveMemory:
    def __init__(self, config: Optional[CognitiveMemoryConfig] = None, seed: int = 0, device="cpu"):
        self.config = config or CognitiveMemoryConfig()
        self.episodic = EpisodicMemory(self.config.episodic, device, seed)
        self.semantic = SemanticMemory(self.config.semantic, device)
        self.working = WorkingMemory(self.config.working, device)
        self.procedural = ProceduralMemory(self.config.procedural, device)
        self.device = device

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """[1, n + slot_dim + embedding_dim + skill_dim]: the input, the attended working memory after writing the
        input to slot 0, the mean of the (up to) 3 nearest concepts, and the recalled skill (zeros where a store
        has nothing)."""
        c = self.config
        flat = x.reshape(-1).float().to(self.device)
        self.working.write(0, flat)
        attended = self.working.attend(flat)
        near, _ = self.semantic.retrieve(flat, 3)
        sem = near.mean(0) if near.shape[0] else torch.zeros(c.semantic.embedding_dim, device=self.device)
        skill = self.procedural.recall(flat)
        if skill is None:
            skill = torch.zeros(c.procedural.skill_dim, device=self.device)
        return torch.cat([flat, attended, sem, skill]).unsqueeze(0)

    __call__ = forward

    def record(self, state, action, reward, next_state):
        if self.episodic.record(state, action, reward, next_state):
            self.consolidate()

    def consolidate(self, top: int = 8) -> int:
        """Episodic -> semantic: the highest-priority transitions become concepts keyed by their buffer index."""
        idx = sorted(range(len(self.episodic)), key=lambda i: -self.episodic.priority[i])[:top]
        for i in idx:
            self.semantic.store(1_000_000 + i, self.episodic.items[i][0])
        return len(idx)

    def num_params(self) -> int:
        c = self.config
        return (c.semantic.max_concepts * c.semantic.embedding_dim + c.working.num_slots * c.working.slot_dim
                + c.procedural.cache_size * (c.procedural.state_dim + c.procedural.skill_dim))

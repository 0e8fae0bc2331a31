"""Cognitive memory stores and their combined forward pass."""
import torch

from sneppx_alg_b200.algorithms.cognition import (CognitiveMemory, CognitiveMemoryConfig, EpisodicConfig, ProceduralConfig,
                                                  SemanticConfig, WorkingConfig)


def _cfg():
    return CognitiveMemoryConfig(EpisodicConfig(capacity=4, max_priority_samples=3, consolidation_interval=3),
                                 SemanticConfig(max_concepts=3, max_edges=2, embedding_dim=8, lru_size=2),
                                 WorkingConfig(num_slots=3, slot_dim=8), ProceduralConfig(cache_size=2, state_dim=8, skill_dim=4,
                                                                                         compilation_threshold=2))


def test_forward_layout_matches_store_contents():
    m = CognitiveMemory(_cfg())
    x = torch.arange(8.0)
    out = m(x)
    assert out.shape == (1, 8 + 8 + 8 + 4)
    assert torch.equal(out[0, :8], x) and torch.allclose(out[0, 8:16], x)  # one valid slot: attention returns it
    assert torch.count_nonzero(out[0, 16:]) == 0
    m.semantic.store(1, x)
    m.semantic.store(2, -x)
    m.procedural.learn(x, torch.ones(4))
    out = m(x)
    assert torch.allclose(out[0, 16:24], torch.zeros(8))  # mean of x and -x
    assert torch.equal(out[0, 24:], torch.ones(4))


def test_working_memory_attention_weights():
    m = CognitiveMemory(_cfg())
    a, b = torch.zeros(8), torch.zeros(8)
    a[0], b[1] = 10.0, 10.0
    m.working.write(1, a)
    m.working.write(2, b)
    got = m.working.attend(a)
    w = torch.softmax(torch.tensor([100.0, 0.0]) / 8 ** 0.5, 0)
    assert torch.allclose(got, w[0] * a + w[1] * b, atol=1e-5)
    assert m.working.read(0) is None and torch.equal(m.working.read(1), a)
    m.working.clear()
    assert torch.count_nonzero(m.working.attend(a)) == 0


def test_semantic_lru_eviction_and_relations():
    s = CognitiveMemory(_cfg()).semantic
    e = torch.eye(8)
    for i in range(3):
        s.store(i, e[i])
    assert s.relate(0, 1, 0.5) and s.relate(1, 2) and not s.relate(0, 2)  # edge budget is 2
    assert not s.relate(0, 9) and s.neighbours(1) == {0: 0.5, 2: 1.0}
    _, ids = s.retrieve(e[0], 1)  # touches concept 0
    assert ids == [0]
    s.store(3, e[3])  # evicts the least recently used: concept 1, with its relations
    assert 1 not in s.slot and s.edges == {} and set(s.slot) == {0, 2, 3}
    assert s.forget(2) and not s.forget(2)
    emb, ids = s.retrieve(e[3] + 0.1 * e[0], 5)
    assert ids == [3, 0] and emb.shape == (2, 8)


def test_episodic_ring_priority_and_consolidation():
    m = CognitiveMemory(_cfg(), seed=1)
    e = torch.eye(8)
    for i in range(6):
        m.record(e[i], torch.zeros(2), reward=float(i), next_state=e[i])
    ep = m.episodic
    assert len(ep) == 4 and ep.recorded == 6
    assert {float(r) for _, _, r, _ in ep.items} == {2.0, 3.0, 4.0, 5.0}
    (idx, sim), = ep.retrieve(e[5], 1)
    assert sim > 0.99 and ep.items[idx][2] == 5.0
    picks = ep.sample(10)
    assert len(picks) == 3 and len(set(picks)) == 3
    # records 3 and 6 hit the consolidation interval: concepts exist in semantic memory
    assert len(m.semantic.slot) > 0


def test_procedural_compile_and_eviction():
    p = CognitiveMemory(_cfg()).procedural
    e = torch.eye(8)
    p.learn(e[0], torch.full((4,), 1.0))
    p.learn(e[1], torch.full((4,), 2.0))
    assert p.recall(e[2]) is None
    for _ in range(2):
        assert torch.equal(p.recall(e[0]), torch.full((4,), 1.0))
    assert p.compile() == 1 and p.compiled_states.shape == (1, 8) and len(p.states) == 1
    p.learn(e[2], torch.full((4,), 3.0))
    p.learn(e[3], torch.full((4,), 4.0))  # cache of 2 is full: the unused pair for e[1] goes
    assert torch.equal(p.recall(e[0]), torch.full((4,), 1.0))  # compiled skills survive eviction
    assert p.recall(e[1]) is None

"""Continuous-batching inference engine with a paged KV cache (real KV reuse, chunked prefill, prefix caching).

Each ``step()`` admits waiting requests while KV blocks and batch slots allow (FCFS or priority), prefills at
most ``max_prefill_tokens`` prompt tokens (one sequence at a time through the flash-attention kernel, writing K/V
into the block pool), then decodes one token for every running sequence in a single batch through the paged decode
kernel. The reference's scheduler has the same admission rules (max_batch_size 32, FCFS / priority;
interface_bindings/continuous_batching.py:64-179) but re-runs the whole prefix every token; its C serving engine
(net/http/serving_engine.c) holds the queue / metrics logic mirrored in ``csrc/host/serving_core.cpp``.
"""
from __future__ import annotations

import heapq
import itertools
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import torch

from ..ops import functional as ops
from ..ops import paged
from .generation import apply_repetition_penalty, sample_from_logits
from .kv_cache import PagedKVCache


@dataclass
class SamplingParams:
    max_new_tokens: int = 64
    do_sample: bool = False
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    eos_token_id: Optional[int] = None
    stop_token_ids: tuple = ()
    stop_fn: Optional[Callable[[List[int]], bool]] = None   # called with the output so far; True ends the request


@dataclass(order=True)
class Request:
    priority: int
    arrival: float
    req_id: int = field(compare=False)
    prompt: List[int] = field(compare=False)
    params: SamplingParams = field(compare=False, default_factory=SamplingParams)
    output: List[int] = field(compare=False, default_factory=list)
    prefilled: int = field(compare=False, default=0)
    first_token_time: Optional[float] = field(compare=False, default=None)
    finish_time: Optional[float] = field(compare=False, default=None)
    on_token: Optional[Callable] = field(compare=False, default=None)

    @property
    def tokens(self):
        return self.prompt + self.output


class LlamaPagedRunner:
    """Runs a Llama-family model (``models/llama.py``) against the paged cache: fused QKV GEMM -> RoPE + cache append
    kernel -> flash attention (prefill) or paged decode attention -> rest of the block."""

    def __init__(self, model, cache: PagedKVCache):
        self.model, self.cache = model, cache
        cfg = model.config
        self.H, self.Hk, self.D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim

    def _layers(self, x, attn_fn):
        m = self.model
        delta, resid = x, None
        for li, layer in enumerate(m.layers):
            if resid is None:
                h, resid = layer.attn_norm(delta), delta
            else:
                h, resid = layer.attn_norm(delta, residual=resid)
            qkv = layer.attn.qkv_proj(h)
            o = attn_fn(li, qkv)
            a = layer.attn.o_proj(o)
            h, resid = layer.mlp_norm(a, residual=resid)
            delta = layer.mlp(h)
        h, _ = m.norm(delta, residual=resid)
        return h

    @torch.no_grad()
    def prefill(self, seq_id: int, tokens: List[int], start: int):
        """Process prompt tokens [start, len) of one sequence; returns logits of the last position."""
        m, H, Hk, D = self.model, self.H, self.Hk, self.D
        dev = m.embedding.weight.device
        ids = torch.tensor(tokens[start:], dtype=torch.long, device=dev)
        T = ids.numel()
        slots = torch.tensor(self.cache.reserve(seq_id, T), dtype=torch.int32, device=dev)
        pos = torch.arange(start, start + T, dtype=torch.int32, device=dev)
        cos, sin = m.rope(dev, start + T)

        def attn(li, qkv):
            q2 = qkv.view(T, (H + 2 * Hk) * D)
            paged.kv_append_(q2, cos, sin, pos, slots, self.cache.k[li], self.cache.v[li], H, Hk, D)
            q = q2[:, : H * D].view(1, T, H, D)
            if start == 0:
                k = q2[:, H * D: (H + Hk) * D].view(1, T, Hk, D)
                v = q2[:, (H + Hk) * D:].view(1, T, Hk, D)
            else:   # later chunk / cached prefix: keys and values of the whole sequence come from the pool
                kk, vv = self.cache.gather(li, seq_id, start + T)
                k, v = kk.unsqueeze(0), vv.unsqueeze(0)
            return ops.attention(q, k, v, causal=True).reshape(1, T, H * D)

        h = self._layers(m.embedding(ids).unsqueeze(0), attn)
        return ops.linear(h[:, -1], m.head_weight()).float()

    @torch.no_grad()
    def prefill_batch(self, seq_ids: List[int], prompts: List[List[int]]):
        """Whole prompts of EQUAL length (nothing cached) in one pass: the GEMMs see n x T rows and the attention
        kernel a batch of n; returns the logits of the last position of every sequence [n, V]."""
        m, H, Hk, D = self.model, self.H, self.Hk, self.D
        dev = m.embedding.weight.device
        n, T = len(prompts), len(prompts[0])
        assert all(len(p) == T for p in prompts)
        ids = torch.tensor(prompts, dtype=torch.long, device=dev)
        slots = torch.tensor([s for sid in seq_ids for s in self.cache.reserve(sid, T)], dtype=torch.int32, device=dev)
        pos = torch.arange(T, dtype=torch.int32, device=dev).repeat(n)
        cos, sin = m.rope(dev, T)

        def attn(li, qkv):
            q2 = qkv.view(n * T, (H + 2 * Hk) * D)
            paged.kv_append_(q2, cos, sin, pos, slots, self.cache.k[li], self.cache.v[li], H, Hk, D)
            q3 = q2.view(n, T, (H + 2 * Hk) * D)
            q = q3[..., : H * D].view(n, T, H, D)
            k = q3[..., H * D: (H + Hk) * D].view(n, T, Hk, D)
            v = q3[..., (H + Hk) * D:].view(n, T, Hk, D)
            return ops.attention(q, k, v, causal=True).reshape(n, T, H * D)

        h = self._layers(m.embedding(ids), attn)
        return ops.linear(h[:, -1], m.head_weight()).float()

    # ------------------------------------------------------------------ decode
    def enable_graphs(self, max_batch: int, max_len: int):
        """Capture the decode step into CUDA graphs, one per batch-size bucket (1, 2, 4, .. max_batch): a decode step
        is some 300 small launches for a few microseconds of work each, so replaying one graph instead of launching
        them from Python removes most of the step time. Inputs live in one static int32 buffer (token ids, positions,
        KV slots, sequence lengths, block table of ``max_len`` tokens per sequence) filled with a single host -> device
        copy per step; padding rows have slot -1 and length 0 and touch nothing."""
        dev = self.model.embedding.weight.device
        if dev.type != "cuda":
            return
        bs = self.cache.block_size
        self._g_max_blocks = (max_len + bs - 1) // bs
        self._g_max_len = self._g_max_blocks * bs
        self._g_buckets = []
        b = 1
        while b < max_batch:
            self._g_buckets.append(b)
            b *= 2
        self._g_buckets.append(max_batch)
        self._graphs = {}
        self.model.rope(dev, self._g_max_len)

    def _decode_body(self, B, ids, pos, slots, bt, lens):
        m, H, Hk, D = self.model, self.H, self.Hk, self.D
        cos, sin = m.rope(ids.device, self._g_max_len if getattr(self, "_graphs", None) is not None else int(pos.max()) + 1)

        def attn(li, qkv):
            q2 = qkv.view(B, (H + 2 * Hk) * D)
            paged.kv_append_(q2, cos, sin, pos, slots, self.cache.k[li], self.cache.v[li], H, Hk, D)
            q = q2[:, : H * D].view(B, H, D)
            return paged.paged_decode(q, self.cache.k[li], self.cache.v[li], bt, lens).reshape(B, 1, H * D)

        from ..ops.gemm import static_weights
        with static_weights():     # weights are not written while serving: decode GEMMs may prefetch them early
            h = self._layers(m.embedding(ids).unsqueeze(1), attn)
            return ops.linear(h[:, -1], m.head_weight()).float()

    def _graph_for(self, Bb):
        g = self._graphs.get(Bb)
        if g is not None:
            return g
        dev = self.model.embedding.weight.device
        mb = self._g_max_blocks
        n = 4 * Bb + Bb * mb
        host = torch.zeros(n, dtype=torch.int32).pin_memory()
        buf = torch.zeros(n, dtype=torch.int32, device=dev)
        views = dict(ids=buf[:Bb], pos=buf[Bb:2 * Bb], slots=buf[2 * Bb:3 * Bb], lens=buf[3 * Bb:4 * Bb],
                     bt=buf[4 * Bb:].view(Bb, mb))
        # warm-up outside the graph with rows that write nothing (slot -1, length 0), then capture
        buf[2 * Bb:3 * Bb].fill_(-1)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self._decode_body(Bb, views["ids"], views["pos"], views["slots"], views["bt"], views["lens"])
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):   # other threads (HTTP handlers) may call CUDA
            out = self._decode_body(Bb, views["ids"], views["pos"], views["slots"], views["bt"], views["lens"])
        g = self._graphs[Bb] = dict(graph=graph, host=host, buf=buf, out=out, hv=host.numpy())
        return g

    @torch.no_grad()
    def decode(self, seq_ids: List[int], last_tokens: List[int]):
        """One token for each running sequence; returns logits [B, V]."""
        m = self.model
        dev = m.embedding.weight.device
        B = len(seq_ids)
        pos_list = [self.cache.lens[s] for s in seq_ids]
        slot_list = [self.cache.reserve(s, 1)[0] for s in seq_ids]
        graphs = getattr(self, "_graphs", None)
        if graphs is not None and B <= self._g_buckets[-1] and max(pos_list) + 1 <= self._g_max_len:
            Bb = next(b for b in self._g_buckets if b >= B)
            g = self._graph_for(Bb)
            hv, mb = g["hv"], self._g_max_blocks
            hv[:4 * Bb] = 0
            hv[2 * Bb:3 * Bb] = -1
            hv[:B] = last_tokens
            hv[Bb:Bb + B] = pos_list
            hv[2 * Bb:2 * Bb + B] = slot_list
            hv[3 * Bb:3 * Bb + B] = [p + 1 for p in pos_list]
            bt = hv[4 * Bb:].reshape(Bb, mb)
            for i, s in enumerate(seq_ids):
                t = self.cache.tables[s]
                bt[i, :len(t)] = t
            g["buf"].copy_(g["host"], non_blocking=True)
            g["graph"].replay()
            return g["out"][:B]
        slots = torch.tensor(slot_list, dtype=torch.int32, device=dev)
        pos = torch.tensor(pos_list, dtype=torch.int32, device=dev)
        bt, lens = self.cache.block_table_tensor(seq_ids, dev)
        ids = torch.tensor(last_tokens, dtype=torch.long, device=dev)
        saved, self._graphs = graphs, None          # eager step: rope tables sized by the longest sequence
        try:
            return self._decode_body(B, ids, pos, slots, bt, lens)
        finally:
            self._graphs = saved


class TPLlamaPagedRunner(LlamaPagedRunner):
    """Tensor-parallel form of the paged runner: every rank holds H / tp query heads and Hk / tp key-value heads (and
    their slice of the paged cache), 1 / tp of the MLP's hidden units, and the replicated embedding, norms and LM
    head. Two all-reduces per layer (after the attention output projection and after the MLP down projection) make the
    hidden state identical on all ranks, so every rank runs the same scheduler and samples the same tokens. The
    projections are slices of the full weights (views, no copy)."""

    def __init__(self, model, cache: PagedKVCache, group=None):
        import torch.distributed as dist
        super().__init__(model, cache)
        self.group = group if group is not None else dist.group.WORLD
        self.tp, r = dist.get_world_size(self.group), dist.get_rank(self.group)
        H, Hk, D = self.H, self.Hk, self.D
        assert H % self.tp == 0 and Hk % self.tp == 0, "query and key-value heads must divide over the tensor-parallel ranks"
        hl, kl = H // self.tp, Hk // self.tp
        self.local = []
        for layer in model.layers:
            wqkv, wo = layer.attn.qkv_proj.weight, layer.attn.o_proj.weight
            q = wqkv[r * hl * D:(r + 1) * hl * D]
            k = wqkv[H * D + r * kl * D: H * D + (r + 1) * kl * D]
            v = wqkv[(H + Hk) * D + r * kl * D: (H + Hk) * D + (r + 1) * kl * D]
            gu, dn = layer.mlp.gate_up_proj.weight, layer.mlp.down_proj.weight
            ff = gu.shape[0] // 2
            assert ff % self.tp == 0
            fl = ff // self.tp
            self.local.append({"qkv": torch.cat([q, k, v]).contiguous(), "o": wo[:, r * hl * D:(r + 1) * hl * D].contiguous(),
                               "gu": torch.cat([gu[r * fl:(r + 1) * fl], gu[ff + r * fl: ff + (r + 1) * fl]]).contiguous(),
                               "down": dn[:, r * fl:(r + 1) * fl].contiguous(), "act": layer.mlp.act})
        self.H, self.Hk = hl, kl
        # all-reduce of the layer outputs: this package's peer-load kernel for messages up to 4 MiB (every decode
        # step, short prefill chunks), NCCL above that. The kernel keeps its epoch on the device: graph-capturable.
        self._sg = self._stage = None
        p = model.embedding.weight
        if p.is_cuda and p.dtype == torch.bfloat16 and dist.get_backend(self.group) == "nccl" and self.tp > 1:
            from ..parallel.symm import SymmGroup
            self._sg = SymmGroup(self.group)
            self._stage = self._sg.alloc(2 << 20, torch.bfloat16)
            self._ar_state = torch.zeros(2, dtype=torch.int32, device=p.device)
            torch.cuda.synchronize()
            dist.barrier(self.group)

    def _all_reduce(self, t):
        import torch.distributed as dist
        if self._sg is not None and t.numel() <= self._stage.tensor.numel() and t.numel() % 8 == 0:
            return self._sg.allreduce_bf16_(t if t.is_contiguous() else t.contiguous(), self._stage, self._ar_state)
        dist.all_reduce(t, group=self.group)
        return t

    def _layers(self, x, attn_fn):
        m = self.model
        delta, resid = x, None
        for li, (layer, w) in enumerate(zip(m.layers, self.local)):
            if resid is None:
                h, resid = layer.attn_norm(delta), delta
            else:
                h, resid = layer.attn_norm(delta, residual=resid)
            o = attn_fn(li, ops.linear(h, w["qkv"]))
            a = self._all_reduce(ops.linear(o, w["o"]))
            h, resid = layer.mlp_norm(a, residual=resid)
            delta = self._all_reduce(ops.linear(ops.glu(ops.linear(h, w["gu"]), w["act"]), w["down"]))
        h, _ = m.norm(delta, residual=resid)
        return h


class _Slots:
    def __init__(self, n):
        self.num_free = n


class StateCache:
    """Admission bookkeeping for models whose per-sequence memory is a fixed-size recurrent state (Mamba-2 / HSS):
    one slot per running sequence instead of KV blocks. Offers the few calls the engine makes on a cache."""

    block_size = 1 << 30   # any request needs one "block"

    def __init__(self, max_sequences: int, on_free=None):
        self.pool = _Slots(max_sequences)
        self._live, self._on_free = set(), on_free

    def available_blocks(self):
        return self.pool.num_free

    def make_room(self, n):
        return self.pool.num_free >= n

    def add_sequence(self, seq_id, prompt):
        self.pool.num_free -= 1
        self._live.add(seq_id)
        return 0   # no prefix reuse: the state after a prefix is not kept

    def free_sequence(self, seq_id, tokens=None):
        if seq_id in self._live:
            self._live.discard(seq_id)
            self.pool.num_free += 1
            if self._on_free:
                self._on_free(seq_id)


class StatefulRunner:
    """Runs any model that follows the generation contract ``forward(input_ids, past_key_values, use_cache) ->
    {"logits", "past_key_values"}`` with a per-layer state of tensors batched along dim 0 (``Mamba2ForCausalLM``: a
    list of {"conv", "ssm"} dicts). Prefill runs one sequence; decode stacks the states of all running sequences,
    advances them together by one token, and splits them again."""

    def __init__(self, model):
        self.model = model
        self.states = {}

    def release(self, seq_id):
        self.states.pop(seq_id, None)

    @torch.no_grad()
    def prefill(self, seq_id: int, tokens: List[int], start: int):
        dev = next(self.model.parameters()).device
        ids = torch.tensor(tokens[start:], dtype=torch.long, device=dev).unsqueeze(0)
        out = self.model(ids, use_cache=True)
        self.states[seq_id] = out["past_key_values"]
        return out["logits"][:, -1].float()

    @staticmethod
    def _stack(states):
        first = states[0]
        return [{k: (None if first[li][k] is None else torch.cat([s[li][k] for s in states], dim=0)) for k in first[li]}
                for li in range(len(first))]

    @torch.no_grad()
    def decode(self, seq_ids: List[int], last_tokens: List[int]):
        dev = next(self.model.parameters()).device
        batched = self._stack([self.states[s] for s in seq_ids])
        ids = torch.tensor(last_tokens, dtype=torch.long, device=dev).unsqueeze(1)
        out = self.model(ids, past_key_values=batched, use_cache=True)
        new = out["past_key_values"]
        for b, s in enumerate(seq_ids):
            self.states[s] = [{k: (None if v is None else v[b:b + 1].clone()) for k, v in layer.items()} for layer in new]
        return out["logits"][:, -1].float()


class LLMEngine:
    def __init__(self, model, num_blocks=2048, block_size=16, max_batch_size=32, max_prefill_tokens=8192,
                 policy="fcfs", enable_prefix_cache=True, runner=None, tp_group=None, cuda_graphs=True,
                 max_model_len=None):
        cfg = model.config
        p = next(model.parameters())
        if runner is None and getattr(cfg, "architecture", "transformer") == "mamba2":
            runner = StatefulRunner(model)   # recurrent-state models: no KV cache, one state slot per sequence
        if isinstance(runner, StatefulRunner):
            self.cache = StateCache(max_batch_size, on_free=runner.release)
        elif tp_group is not None:
            import torch.distributed as dist
            tp = dist.get_world_size(tp_group)
            self.cache = PagedKVCache(cfg.num_hidden_layers, num_blocks, block_size, cfg.num_key_value_heads // tp, cfg.head_dim,
                                      dtype=p.dtype, device=p.device, enable_prefix_cache=enable_prefix_cache)
            runner = TPLlamaPagedRunner(model, self.cache, tp_group)
        else:
            self.cache = PagedKVCache(cfg.num_hidden_layers, num_blocks, block_size, cfg.num_key_value_heads, cfg.head_dim,
                                      dtype=p.dtype, device=p.device, enable_prefix_cache=enable_prefix_cache)
        self.runner = runner or LlamaPagedRunner(model, self.cache)
        # CUDA-graph decode: the single-GPU runner, and the tensor-parallel runner when its all-reduce is the
        # graph-capturable peer-load kernel
        if cuda_graphs and p.is_cuda and (type(self.runner) is LlamaPagedRunner or getattr(self.runner, "_sg", None) is not None):
            limit = max_model_len or min(getattr(cfg, "max_position_embeddings", 4096) or 4096, num_blocks * block_size)
            self.runner.enable_graphs(max_batch_size, limit)
        self.max_batch_size, self.max_prefill_tokens, self.policy = max_batch_size, max_prefill_tokens, policy
        self.waiting: List[Request] = []
        self.running: Dict[int, Request] = {}
        self.finished: Dict[int, Request] = {}
        self._ids = itertools.count()
        self.generator = None
        self.stats = {"prefill_tokens": 0, "decode_tokens": 0, "cached_prefix_tokens": 0, "steps": 0, "rejected": 0}
        self.failed: Dict[int, str] = {}

    # ------------------------------------------------------------------ API
    def submit(self, prompt: List[int], params: Optional[SamplingParams] = None, priority: int = 0, on_token=None) -> int:
        rid = next(self._ids)
        req = Request(priority if self.policy == "priority" else 0, time.perf_counter(), rid, list(prompt),
                      params or SamplingParams(), on_token=on_token)
        heapq.heappush(self.waiting, req)
        return rid

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _blocks_needed(self, req: Request) -> int:
        bs = self.cache.block_size
        return (len(req.prompt) + req.params.max_new_tokens + bs - 1) // bs

    def _committed(self) -> int:
        """Blocks the running sequences may still claim before they finish (admission keeps these in hand, so a
        decode step never finds the pool empty)."""
        tables = getattr(self.cache, "tables", None)
        if tables is None:
            return 0
        return sum(max(0, self._blocks_needed(r) - len(tables.get(r.req_id, ()))) for r in self.running.values())

    def _fail(self, req: Request, why: str):
        req.finish_time = time.perf_counter()
        self.failed[req.req_id] = why
        self.finished[req.req_id] = req
        self.stats["rejected"] += 1

    @staticmethod
    def _plain_greedy(req: Request) -> bool:
        return not req.params.do_sample and req.params.repetition_penalty == 1.0

    def _emit(self, req: Request, logits_row, tok: Optional[int] = None):
        """`tok`: token already chosen for this row (the batched greedy path picks all rows with one argmax and one
        device-to-host copy instead of one per request)."""
        p = req.params
        if tok is None:
            hist = torch.tensor(req.tokens, device=logits_row.device).unsqueeze(0)
            lg = apply_repetition_penalty(logits_row.unsqueeze(0), hist, p.repetition_penalty)
            tok = int(sample_from_logits(lg, p.do_sample, p.temperature, p.top_k, p.top_p, self.generator)[0])
        now = time.perf_counter()
        if req.first_token_time is None:
            req.first_token_time = now
        req.output.append(tok)
        if req.on_token:
            req.on_token(req.req_id, tok)
        stop = (p.eos_token_id is not None and tok == p.eos_token_id) or tok in p.stop_token_ids \
            or (p.stop_fn is not None and p.stop_fn(req.output))
        if stop or len(req.output) >= p.max_new_tokens:
            req.finish_time = now
            self.cache.free_sequence(req.req_id, req.tokens)
            self.running.pop(req.req_id, None)
            self.finished[req.req_id] = req

    def _admit_same_length(self, first: "Request", budget: int) -> List["Request"]:
        """Pops the waiting requests that can join ``first``'s prefill pass: they are next in queue order, have a
        prompt of the same length, hit no cached prefix, fit the batch, the token budget and the block pool."""
        out, T = [], len(first.prompt)
        reserved = self._blocks_needed(first)
        while self.waiting and len(self.running) + 1 + len(out) < self.max_batch_size and budget >= T and len(out) < 15:
            nxt = self.waiting[0]
            if len(nxt.prompt) != T:
                break
            need = reserved + self._blocks_needed(nxt) + self._committed()
            if need > self.cache.available_blocks() or not self.cache.make_room(need):
                break
            if self.cache.add_sequence(nxt.req_id, nxt.prompt) != 0:     # a cached prefix: it prefills on its own
                self.cache.free_sequence(nxt.req_id)
                break
            heapq.heappop(self.waiting)
            out.append(nxt)
            reserved += self._blocks_needed(nxt)
            budget -= T
        return out

    def step(self):
        """One scheduler iteration: admit + prefill, then one decode step for all running sequences."""
        self.stats["steps"] += 1
        budget = self.max_prefill_tokens
        while self.waiting and len(self.running) < self.max_batch_size and budget > 0:
            req = self.waiting[0]
            need = self._blocks_needed(req) + self._committed()
            if need > self.cache.available_blocks() or not self.cache.make_room(need):
                total = getattr(self.cache.pool, "num_blocks", None)
                if not self.running and (total is None or self._blocks_needed(req) > total
                                         or need > self.cache.available_blocks()):
                    # nothing will ever free more room for it: fail it instead of waiting forever
                    heapq.heappop(self.waiting)
                    self._fail(req, "request needs more KV blocks than the pool can ever provide")
                    continue
                break
            heapq.heappop(self.waiting)
            cached = self.cache.add_sequence(req.req_id, req.prompt)
            self.stats["cached_prefix_tokens"] += cached
            group = [req]
            if cached == 0 and hasattr(self.runner, "prefill_batch"):
                # requests behind it with a prompt of the same length (and nothing cached) share the pass
                group += self._admit_same_length(req, budget - len(req.prompt))
            if len(group) > 1:
                logits = self.runner.prefill_batch([g.req_id for g in group], [g.prompt for g in group])
                picks = logits.argmax(dim=-1).tolist() if any(self._plain_greedy(g) for g in group) else None
            else:
                logits = self.runner.prefill(req.req_id, req.prompt, cached)
                picks = [int(logits[0].argmax())] if self._plain_greedy(req) else None
            for i, g in enumerate(group):
                n = len(g.prompt) - (cached if i == 0 else 0)
                budget -= n
                self.stats["prefill_tokens"] += n
                self.running[g.req_id] = g
                self._emit(g, logits[i], picks[i] if picks is not None and self._plain_greedy(g) else None)
        active = [r for r in self.running.values() if r.output]
        if active:
            ids = [r.req_id for r in active]
            logits = self.runner.decode(ids, [r.output[-1] for r in active])
            self.stats["decode_tokens"] += len(active)
            greedy = logits.argmax(dim=-1).tolist() if any(self._plain_greedy(r) for r in active) else None
            for i, (r, row) in enumerate(zip(active, logits)):
                self._emit(r, row, greedy[i] if greedy is not None and self._plain_greedy(r) else None)

    def run_until_done(self, max_steps: int = 1_000_000):
        n = 0
        while self.has_work() and n < max_steps:
            self.step()
            n += 1
        return self.finished

    def generate(self, prompts: List[List[int]], params: Optional[SamplingParams] = None) -> List[List[int]]:
        ids = [self.submit(p, params) for p in prompts]
        self.run_until_done()
        return [self.finished[i].output for i in ids]

"""Llama-family decoder (LLaMA-2/3, Mistral, Qwen2): RMSNorm -> GQA attention with RoPE -> RMSNorm
-> SwiGLU, with the residual adds fused into the norms, one GEMM for Q|K|V and one for gate|up.

API of the reference's ``LlamaForCausalLM`` (interface_bindings/llama_models.py:285-420):
``forward(input_ids, attention_mask=None, position_ids=None, past_key_values=None, use_cache=False,
labels=None)`` returning a dict with ``logits`` / ``loss`` / ``past_key_values``. Parameter names
map one-to-one onto the reference's checkpoint names (``layers.{i}.attn.q_proj.weight`` ...;
model_zoo.py:1049-1158) through ``to_reference_state_dict`` / ``load_reference_state_dict``.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as tnn

from ..nn.modules import Embedding, Linear, Module, RMSNorm
from ..ops import functional as ops
from .config import ModelConfig, config_from_name


class LlamaAttention(Module):
    def __init__(self, cfg: ModelConfig, dtype=None, device=None):
        super().__init__()
        self.H, self.Hk, self.D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        self.window = cfg.sliding_window
        d = cfg.hidden_size
        self.qkv_proj = Linear(d, (self.H + 2 * self.Hk) * self.D, bias=False, dtype=dtype, device=device,
                               init_std=cfg.initializer_range)
        self.o_proj = Linear(self.H * self.D, d, bias=False, dtype=dtype, device=device,
                             init_std=cfg.initializer_range)

    def forward(self, x, rope, positions=None, kv_cache=None):
        B, S, _ = x.shape
        H, Hk, D = self.H, self.Hk, self.D
        qkv = self.qkv_proj(x)
        qkv = ops.rope_qk_(qkv, rope[0], rope[1], H + Hk, D, positions)
        q = qkv[..., : H * D].view(B, S, H, D)
        k = qkv[..., H * D: (H + Hk) * D].view(B, S, Hk, D)
        v = qkv[..., (H + Hk) * D:].view(B, S, Hk, D)
        if kv_cache is not None:
            k, v = kv_cache.append(k, v)
        o = ops.attention(q, k, v, causal=True, window=self.window)
        return self.o_proj(o.reshape(B, S, H * D))


class LlamaMLP(Module):
    def __init__(self, cfg: ModelConfig, dtype=None, device=None, d_ff=None):
        super().__init__()
        d_ff = d_ff or cfg.intermediate_size
        self.act = cfg.ffn_act if cfg.ffn_act in ops.GLU_ACT else "silu"
        self.gate_up_proj = Linear(cfg.hidden_size, 2 * d_ff, bias=False, dtype=dtype, device=device,
                                   init_std=cfg.initializer_range)
        self.down_proj = Linear(d_ff, cfg.hidden_size, bias=False, dtype=dtype, device=device,
                                init_std=cfg.initializer_range)

    def forward(self, x):
        return self.down_proj(ops.glu(self.gate_up_proj(x), self.act))


class LlamaBlock(Module):
    def __init__(self, cfg: ModelConfig, dtype=None, device=None):
        super().__init__()
        self.attn_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype=dtype, device=device)
        self.attn = LlamaAttention(cfg, dtype, device)
        self.mlp_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype=dtype, device=device)
        self.mlp = LlamaMLP(cfg, dtype, device)

    def forward(self, delta, resid, rope, positions=None, kv_cache=None):
        """(delta, resid): the residual stream is resid + delta; the add happens inside the norm kernel."""
        if resid is None:
            h, resid = self.attn_norm(delta), delta
        else:
            h, resid = self.attn_norm(delta, residual=resid)
        a = self.attn(h, rope, positions, kv_cache)
        h, resid = self.mlp_norm(a, residual=resid)
        return self.mlp(h), resid


class KVCache:
    """Contiguous per-layer KV cache for incremental decoding ([B, max_len, Hk, D])."""

    def __init__(self, B, max_len, Hk, D, dtype, device):
        self.k = torch.empty(B, max_len, Hk, D, dtype=dtype, device=device)
        self.v = torch.empty(B, max_len, Hk, D, dtype=dtype, device=device)
        self.len = 0

    def append(self, k, v):
        S = k.shape[1]
        self.k[:, self.len: self.len + S] = k
        self.v[:, self.len: self.len + S] = v
        self.len += S
        return self.k[:, : self.len], self.v[:, : self.len]


class LlamaForCausalLM(Module):
    def __init__(self, cfg: ModelConfig, dtype=None, device=None, with_head: bool = True):
        super().__init__()
        self.config = cfg
        d = cfg.hidden_size
        self.embedding = Embedding(cfg.vocab_size, d, dtype=dtype, device=device, init_std=cfg.initializer_range)
        self.layers = tnn.ModuleList([LlamaBlock(cfg, dtype, device) for _ in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(d, cfg.rms_norm_eps, dtype=dtype, device=device)
        if cfg.tie_word_embeddings or not with_head:
            self.lm_head = None
        else:
            self.lm_head = Linear(d, cfg.vocab_size, bias=False, dtype=dtype, device=device,
                                  init_std=cfg.initializer_range)
        self._rope = None
        self.activation_checkpointing = False

    # ------------------------------------------------------------------ helpers
    def rope(self, device, need):
        cfg = self.config
        if self._rope is None or self._rope[0].device != torch.device(device) or self._rope[0].shape[0] < need:
            n = max(need, cfg.max_position_embeddings or need)
            scaling = cfg.rope_scaling if isinstance(cfg.rope_scaling, str) else None
            self._rope = ops.rope_tables(n, cfg.head_dim, cfg.rope_theta, device, scaling, cfg.rope_scale_factor)
        return self._rope

    def head_weight(self):
        return self.embedding.weight if self.lm_head is None else self.lm_head.weight

    def init_kv_cache(self, B, max_len, dtype=None, device=None):
        cfg = self.config
        p = self.embedding.weight
        return [KVCache(B, max_len, cfg.num_key_value_heads, cfg.head_dim, dtype or p.dtype, device or p.device)
                for _ in self.layers]

    # ------------------------------------------------------------------ forward
    def hidden_states(self, input_ids, position_ids=None, past_key_values=None):
        B, S = input_ids.shape
        past = past_key_values[0].len if past_key_values else 0
        rope = self.rope(input_ids.device, past + S)
        if position_ids is None and past:
            position_ids = torch.arange(past, past + S, device=input_ids.device).expand(B, S)
        delta, resid = self.embedding(input_ids), None
        for i, layer in enumerate(self.layers):
            cache = past_key_values[i] if past_key_values else None
            if self.activation_checkpointing and self.training and cache is None:
                from torch.utils.checkpoint import checkpoint
                delta, resid = checkpoint(layer, delta, resid, rope, position_ids, None, use_reentrant=False)
            else:
                delta, resid = layer(delta, resid, rope, position_ids, cache)
        if resid is None:
            return self.norm(delta)
        h, _ = self.norm(delta, residual=resid)
        return h

    def forward(self, input_ids, attention_mask=None, position_ids=None, past_key_values=None, use_cache=False,
                labels=None, shift_labels=True):
        if use_cache and past_key_values is None:
            past_key_values = self.init_kv_cache(input_ids.shape[0], self.config.max_position_embeddings)
        h = self.hidden_states(input_ids, position_ids, past_key_values)
        out = {"past_key_values": past_key_values if use_cache else None}
        if labels is not None:
            if shift_labels:
                tgt = torch.full_like(labels, -100)
                tgt[:, :-1] = labels[:, 1:]
            else:
                tgt = labels
            out["loss"] = ops.linear_cross_entropy(h, self.head_weight(), tgt)
            out["logits"] = None
        else:
            out["logits"] = ops.linear(h, self.head_weight())
        return out

    # ------------------------------------------------------------------ checkpoint name mapping
    def to_reference_state_dict(self):
        """State dict under the reference's tensor names, in its fixed write order (model_zoo.py:1140-1158)."""
        cfg = self.config
        H, Hk, D, F_ = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size
        sd = {"embedding": self.embedding.weight, "norm": self.norm.weight, "lm_head": self.head_weight()}
        for i, l in enumerate(self.layers):
            w = l.attn.qkv_proj.weight
            gu = l.mlp.gate_up_proj.weight
            p = f"layers.{i}."
            sd[p + "attn_norm.weight"] = l.attn_norm.weight
            sd[p + "attn.q_proj.weight"] = w[: H * D]
            sd[p + "attn.k_proj.weight"] = w[H * D: (H + Hk) * D]
            sd[p + "attn.v_proj.weight"] = w[(H + Hk) * D:]
            sd[p + "attn.o_proj.weight"] = l.attn.o_proj.weight
            sd[p + "mlp_norm.weight"] = l.mlp_norm.weight
            sd[p + "mlp.gate_proj.weight"] = gu[:F_]
            sd[p + "mlp.up_proj.weight"] = gu[F_:]
            sd[p + "mlp.down_proj.weight"] = l.mlp.down_proj.weight
        return {k: v.detach() for k, v in sd.items()}

    @torch.no_grad()
    def load_reference_state_dict(self, sd, strict=True):
        missing = []

        def get(name):
            if name in sd:
                return torch.as_tensor(sd[name])
            missing.append(name)
            return None

        def put(dst, src):
            if src is not None:
                dst.copy_(src.to(dst.dtype).view(dst.shape))

        put(self.embedding.weight, get("embedding"))
        put(self.norm.weight, get("norm"))
        if self.lm_head is not None:
            put(self.lm_head.weight, get("lm_head"))
        cfg = self.config
        H, Hk, D, F_ = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size
        for i, l in enumerate(self.layers):
            p = f"layers.{i}."
            put(l.attn_norm.weight, get(p + "attn_norm.weight"))
            put(l.attn.qkv_proj.weight[: H * D], get(p + "attn.q_proj.weight"))
            put(l.attn.qkv_proj.weight[H * D: (H + Hk) * D], get(p + "attn.k_proj.weight"))
            put(l.attn.qkv_proj.weight[(H + Hk) * D:], get(p + "attn.v_proj.weight"))
            put(l.attn.o_proj.weight, get(p + "attn.o_proj.weight"))
            put(l.mlp_norm.weight, get(p + "mlp_norm.weight"))
            put(l.mlp.gate_up_proj.weight[:F_], get(p + "mlp.gate_proj.weight"))
            put(l.mlp.gate_up_proj.weight[F_:], get(p + "mlp.up_proj.weight"))
            put(l.mlp.down_proj.weight, get(p + "mlp.down_proj.weight"))
        if strict and missing:
            raise KeyError(f"missing tensors: {missing[:5]}{'...' if len(missing) > 5 else ''}")
        return missing

    # ------------------------------------------------------------------ generation (greedy, cached)
    @torch.no_grad()
    def generate(self, input_ids, max_new_tokens=32, eos_token_id: Optional[int] = None):
        B, S = input_ids.shape
        cache = self.init_kv_cache(B, S + max_new_tokens)
        out = self.forward(input_ids, past_key_values=cache)
        tokens = [input_ids]
        nxt = out["logits"][:, -1].float().argmax(-1, keepdim=True)
        for _ in range(max_new_tokens):
            tokens.append(nxt)
            if eos_token_id is not None and bool((nxt == eos_token_id).all()):
                break
            out = self.forward(nxt, past_key_values=cache)
            nxt = out["logits"][:, -1].float().argmax(-1, keepdim=True)
        return torch.cat(tokens, dim=1)


class MistralForCausalLM(LlamaForCausalLM):
    """Llama architecture under a Mistral configuration (``sliding_window`` selects the windowed attention kernel)."""


class Qwen2ForCausalLM(LlamaForCausalLM):
    """Llama architecture under a Qwen2 configuration (``attention_bias`` adds the q / k / v biases)."""


class LlamaModel(LlamaForCausalLM):
    """The decoder stack alone (embedding, blocks, final norm): no language-model head is allocated and ``forward``
    returns the final hidden states (reference: interface_bindings/llama_models.py:230)."""

    def __init__(self, cfg: ModelConfig, dtype=None, device=None):
        super().__init__(cfg, dtype, device, with_head=False)

    def head_weight(self):
        raise AttributeError(f"{type(self).__name__} has no language-model head")

    def forward(self, input_ids, attention_mask=None, position_ids=None, past_key_values=None, use_cache=False):
        if use_cache and past_key_values is None:
            past_key_values = self.init_kv_cache(input_ids.shape[0], self.config.max_position_embeddings)
        h = self.hidden_states(input_ids, position_ids, past_key_values)
        return {"last_hidden_state": h, "past_key_values": past_key_values if use_cache else None}

    def generate(self, *a, **k):
        raise AttributeError(f"{type(self).__name__} has no language-model head to generate with")


class MistralModel(LlamaModel):
    """Head-less decoder stack under a Mistral configuration."""


class Qwen2Model(LlamaModel):
    """Head-less decoder stack under a Qwen2 configuration."""


class MistralMLP(LlamaMLP):
    """The SwiGLU feed-forward block; Mistral's is Llama's."""


class Qwen2MLP(LlamaMLP):
    """The SwiGLU feed-forward block; Qwen2's is Llama's."""


class MistralAttention(LlamaAttention):
    """Llama attention under a Mistral config (``sliding_window`` set in the config selects the windowed kernel)."""


class Qwen2Attention(LlamaAttention):
    """Llama attention under a Qwen2 config (``attention_bias`` set in the config adds the q/k/v biases)."""


class MistralDecoderLayer(LlamaBlock):
    """Pre-norm attention + feed-forward block under a Mistral configuration."""


class Qwen2DecoderLayer(LlamaBlock):
    """Pre-norm attention + feed-forward block under a Qwen2 configuration."""


def create_model(name_or_config, dtype=None, device=None, **overrides):
    """Build a causal LM from a preset name or a ModelConfig (the reference's ``create_model``,
    llama_models.py:757)."""
    cfg = name_or_config if isinstance(name_or_config, ModelConfig) else config_from_name(name_or_config)
    for k, v in overrides.items():
        setattr(cfg, k, v)
    cfg.__post_init__()
    from . import build_model
    return build_model(cfg, dtype=dtype, device=device)

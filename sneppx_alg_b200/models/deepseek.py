"""DeepSeek-V2-Lite-shape SER MoE decoder: standard multi-head attention (16 x 128) with RoPE, a dense SwiGLU FFN
in the first layer(s) and SER MoE layers after it (64 routed experts top-6 + 2 shared experts, softmax router with
the load-balance auxiliary loss). The reference's ``DeepSeekV2ForCausalLM`` (interface_bindings/llama_models.py:606)
has MLA projections but dense MLPs only; the MoE layers here are what its preset name implies. ``kv_lora_rank`` /
``q_lora_rank`` from the preset are kept in the config for checkpoint compatibility; attention is plain MHA as the
benchmark config specifies."""
from __future__ import annotations

import torch
import torch.nn as tnn

from ..nn.modules import Embedding, Linear, Module, RMSNorm
from ..nn.moe import SERMoE
from ..ops import functional as ops
from .config import ModelConfig
from .llama import LlamaAttention, LlamaMLP


class DeepSeekLayer(Module):
    def __init__(self, cfg: ModelConfig, dense: bool, dtype=None, device=None, ep_group=None):
        super().__init__()
        d = cfg.hidden_size
        self.attn_norm = RMSNorm(d, cfg.rms_norm_eps, dtype=dtype, device=device)
        self.attn = LlamaAttention(cfg, dtype, device)
        self.mlp_norm = RMSNorm(d, cfg.rms_norm_eps, dtype=dtype, device=device)
        self.is_moe = not dense
        if dense:
            self.mlp = LlamaMLP(cfg, dtype, device)
        else:
            self.mlp = SERMoE(d, cfg.moe_intermediate_size, cfg.num_experts, cfg.num_experts_per_token,
                              cfg.num_shared_experts, cfg.expert_capacity_factor, cfg.router_aux_loss_coef,
                              cfg.router_z_loss_coef, dtype=dtype, device=device, init_std=cfg.initializer_range,
                              ep_group=ep_group, expert_fp8=getattr(cfg, "expert_fp8", False))

    def forward(self, delta, resid, rope, positions=None, kv_cache=None):
        if resid is None:
            h, resid = self.attn_norm(delta), delta
        else:
            h, resid = self.attn_norm(delta, residual=resid)
        a = self.attn(h, rope, positions, kv_cache)
        h, resid = self.mlp_norm(a, residual=resid)
        return self.mlp(h), resid


class DeepSeekV2ForCausalLM(Module):
    def __init__(self, cfg: ModelConfig, dtype=None, device=None, ep_group=None):
        super().__init__()
        self.config = cfg
        self.embedding = Embedding(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device,
                                   init_std=cfg.initializer_range)
        self.layers = tnn.ModuleList([DeepSeekLayer(cfg, i < cfg.first_dense_layers, dtype, device, ep_group)
                                      for i in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype=dtype, device=device)
        self.lm_head = None if cfg.tie_word_embeddings else Linear(cfg.hidden_size, cfg.vocab_size, bias=False,
                                                                   dtype=dtype, device=device,
                                                                   init_std=cfg.initializer_range)
        self._rope = None

    def head_weight(self):
        return self.embedding.weight if self.lm_head is None else self.lm_head.weight

    def rope(self, device, need):
        cfg = self.config
        if self._rope is None or self._rope[0].device != torch.device(device) or self._rope[0].shape[0] < need:
            self._rope = ops.rope_tables(max(need, cfg.max_position_embeddings), cfg.head_dim, cfg.rope_theta, device)
        return self._rope

    def aux_loss(self):
        losses = [l.mlp.aux_loss for l in self.layers if l.is_moe and l.mlp.aux_loss is not None]
        return sum(losses) if losses else 0.0

    def forward(self, input_ids, attention_mask=None, position_ids=None, past_key_values=None, use_cache=False,
                labels=None, shift_labels=True):
        B, S = input_ids.shape
        rope = self.rope(input_ids.device, S)
        delta, resid = self.embedding(input_ids), None
        for layer in self.layers:
            delta, resid = layer(delta, resid, rope, position_ids)
        h, _ = self.norm(delta, residual=resid)
        out = {"past_key_values": None}
        if labels is not None:
            tgt = labels
            if shift_labels:
                tgt = torch.full_like(labels, -100)
                tgt[:, :-1] = labels[:, 1:]
            ce = ops.linear_cross_entropy(h, self.head_weight(), tgt)
            out["ce_loss"] = ce.detach()
            out["loss"] = ce + self.aux_loss()
            out["logits"] = None
        else:
            out["logits"] = ops.linear(h, self.head_weight())
        return out

"""Mamba-2 pure-SSM language model (HSS family): embedding -> N x (RMSNorm -> Mamba2Block) with residuals ->
RMSNorm -> tied LM head. Shape preset 'mamba2-2.7b': 64 layers, d_model 2560, d_state 128, ngroups 8."""
from __future__ import annotations

import torch
import torch.nn as tnn

from ..nn.modules import Embedding, Linear, Module, RMSNorm
from ..nn.ssm import Mamba2Block
from ..ops import functional as ops
from .config import ModelConfig


class Mamba2Layer(Module):
    def __init__(self, cfg: ModelConfig, dtype=None, device=None):
        super().__init__()
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype=dtype, device=device)
        self.mixer = Mamba2Block(cfg.hidden_size, cfg.ssm_state_size, cfg.ssm_conv_kernel, cfg.ssm_expand,
                                 cfg.ssm_head_dim, cfg.ssm_ngroups, cfg.ssm_chunk_size, eps=cfg.rms_norm_eps,
                                 dtype=dtype, device=device, init_std=cfg.initializer_range)

    def forward(self, delta, resid, state=None):
        if resid is None:
            h, resid = self.norm(delta), delta
        else:
            h, resid = self.norm(delta, residual=resid)
        return self.mixer(h, state), resid


class Mamba2ForCausalLM(Module):
    def __init__(self, cfg: ModelConfig, dtype=None, device=None):
        super().__init__()
        self.config = cfg
        self.vocab_padded = (cfg.vocab_size + 63) // 64 * 64   # the LM-head GEMM wants a multiple of 64
        self.embedding = Embedding(self.vocab_padded, cfg.hidden_size, dtype=dtype, device=device,
                                   init_std=cfg.initializer_range)
        self.layers = tnn.ModuleList([Mamba2Layer(cfg, dtype, device) for _ in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype=dtype, device=device)
        self.lm_head = None if cfg.tie_word_embeddings else Linear(cfg.hidden_size, self.vocab_padded, bias=False,
                                                                   dtype=dtype, device=device,
                                                                   init_std=cfg.initializer_range)

    def head_weight(self):
        return self.embedding.weight if self.lm_head is None else self.lm_head.weight

    def hidden_states(self, input_ids, states=None):
        delta, resid = self.embedding(input_ids), None
        for i, layer in enumerate(self.layers):
            delta, resid = layer(delta, resid, states[i] if states is not None else None)
        h, _ = self.norm(delta, residual=resid) if resid is not None else (self.norm(delta), None)
        return h

    def init_states(self, batch):
        return [l.mixer.allocate_state(batch) for l in self.layers]

    def forward(self, input_ids, attention_mask=None, position_ids=None, past_key_values=None, use_cache=False,
                labels=None, shift_labels=True):
        if use_cache and past_key_values is None:
            past_key_values = self.init_states(input_ids.shape[0])
        h = self.hidden_states(input_ids, past_key_values)
        out = {"past_key_values": past_key_values if use_cache else None}
        if labels is not None:
            tgt = labels
            if shift_labels:
                tgt = torch.full_like(labels, -100)
                tgt[:, :-1] = labels[:, 1:]
            out["loss"] = ops.linear_cross_entropy(h, self.head_weight(), tgt)
            out["logits"] = None
        else:
            out["logits"] = ops.linear(h, self.head_weight())[..., : self.config.vocab_size]
        return out

"""HSS + SER hybrid language model: every layer is RMSNorm -> Mamba-2 SSM block -> RMSNorm -> SER MoE FFN, with
tied embeddings. This is the pipeline the reference strings together as HSS -> SER stages of its unified model
(kernel/arch.c:149-239, 263-373) built from real Mamba-2 / SwiGLU-MoE layers. The tiny preset ('hss_ser-tiny':
vocab 32000, d_model 256, 4 layers, 8 heads x 64, d_state 64, 8 experts top-2 d_ff 512, capacity 1.25) is the CPU
fp32 parity config."""
from __future__ import annotations

import torch
import torch.nn as tnn

from ..nn.modules import Embedding, Linear, Module, RMSNorm
from ..nn.moe import SERMoE
from ..nn.ssm import Mamba2Block
from ..ops import functional as ops
from .config import ModelConfig


class HSSSERLayer(Module):
    def __init__(self, cfg: ModelConfig, dtype=None, device=None, ep_group=None):
        super().__init__()
        d = cfg.hidden_size
        self.ssm_norm = RMSNorm(d, cfg.rms_norm_eps, dtype=dtype, device=device)
        self.ssm = Mamba2Block(d, cfg.ssm_state_size, cfg.ssm_conv_kernel, cfg.ssm_expand, cfg.ssm_head_dim,
                               cfg.ssm_ngroups, cfg.ssm_chunk_size, eps=cfg.rms_norm_eps, dtype=dtype, device=device,
                               init_std=cfg.initializer_range)
        self.moe_norm = RMSNorm(d, cfg.rms_norm_eps, dtype=dtype, device=device)
        self.moe = SERMoE(d, cfg.moe_intermediate_size, cfg.num_experts, cfg.num_experts_per_token,
                          cfg.num_shared_experts, cfg.expert_capacity_factor, cfg.router_aux_loss_coef,
                          cfg.router_z_loss_coef, dtype=dtype, device=device, init_std=cfg.initializer_range,
                          ep_group=ep_group)

    def forward(self, delta, resid):
        if resid is None:
            h, resid = self.ssm_norm(delta), delta
        else:
            h, resid = self.ssm_norm(delta, residual=resid)
        a = self.ssm(h)
        h, resid = self.moe_norm(a, residual=resid)
        return self.moe(h), resid


class HSSSERForCausalLM(Module):
    def __init__(self, cfg: ModelConfig, dtype=None, device=None, ep_group=None):
        super().__init__()
        self.config = cfg
        self.embedding = Embedding(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device,
                                   init_std=cfg.initializer_range)
        self.layers = tnn.ModuleList([HSSSERLayer(cfg, dtype, device, ep_group) for _ in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype=dtype, device=device)
        self.lm_head = None if cfg.tie_word_embeddings else Linear(cfg.hidden_size, cfg.vocab_size, bias=False,
                                                                   dtype=dtype, device=device,
                                                                   init_std=cfg.initializer_range)

    def head_weight(self):
        return self.embedding.weight if self.lm_head is None else self.lm_head.weight

    def aux_loss(self):
        losses = [l.moe.aux_loss for l in self.layers if l.moe.aux_loss is not None]
        return sum(losses) if losses else 0.0

    def forward(self, input_ids, attention_mask=None, position_ids=None, past_key_values=None, use_cache=False,
                labels=None, shift_labels=True):
        delta, resid = self.embedding(input_ids), None
        for layer in self.layers:
            delta, resid = layer(delta, resid)
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

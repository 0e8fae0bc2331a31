"""Unified pipeline model: embed -> MHA(+RoPE) -> HSS -> SER -> ARC -> NPE -> FM, every stage optional
(kernel/arch.c:122-145 defaults, :149-239 create, :263-373 forward, :444-530 train graph; Python ``model.py``
``Model`` / ``ModelConfig``).  Defaults enable attention + HSS only, as the reference does."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn as tnn

from ..nn.modules import Embedding, Linear, Module, MultiheadAttention
from ..ops import functional as ops
from .arc import ARCConfig, ARCLayer
from .fm import FMConfig, FMController
from .hss import HSSConfig, HSSModel
from .npe import NPEConfig, NPELayer
from .ser import SERConfig, SERModel


@dataclass
class ModelConfig:
    input_dim: int = 512
    output_dim: int = 512
    vocab_size: int = 256
    seed: int = 42
    num_heads: int = 8
    rope_base: float = 10000.0
    enable_attention: bool = True
    enable_hss: bool = True
    enable_ser: bool = False
    enable_arc: bool = False
    enable_npe: bool = False
    enable_fm: bool = False
    hss: HSSConfig = field(default_factory=HSSConfig)
    ser: SERConfig = field(default_factory=SERConfig)
    arc: ARCConfig = field(default_factory=ARCConfig)
    npe: NPEConfig = field(default_factory=NPEConfig)
    fm: FMConfig = field(default_factory=FMConfig)


class Model(Module):
    def __init__(self, cfg: ModelConfig = None, dtype=None, device=None, **kw):
        super().__init__()
        cfg = cfg or ModelConfig(**kw)
        self.cfg = cfg
        torch.manual_seed(cfg.seed)
        d = cfg.input_dim
        self.embed = Embedding(cfg.vocab_size, d, dtype=dtype, device=device) if cfg.enable_attention else None
        self.attention = MultiheadAttention(d, cfg.num_heads, causal=True, dtype=dtype, device=device) \
            if cfg.enable_attention else None
        if cfg.enable_hss:
            hc = HSSConfig(**{**cfg.hss.__dict__, "input_dim": d, "output_dim": d})
            self.hss = HSSModel(hc, dtype=dtype, device=device)
        else:
            self.hss = None
        if cfg.enable_ser:
            sc = SERConfig(**{**cfg.ser.__dict__, "input_dim": d, "output_dim": d})
            self.ser = SERModel(sc, dtype=dtype, device=device)
        else:
            self.ser = None
        self.arc = ARCLayer(d, cfg.arc, device=device) if cfg.enable_arc else None
        self.npe = NPELayer(d, 2 * d, cfg=cfg.npe, device=device) if cfg.enable_npe else None
        self.fm = FMController(FMConfig(**{**cfg.fm.__dict__, "memory_dim": d}), device=device) if cfg.enable_fm else None
        self.head = Linear(d, cfg.output_dim, bias=True, dtype=dtype, device=device) if cfg.output_dim != d else None
        self._rope = None
        self.aux_loss = None

    def forward(self, x):
        """x: token ids [B, S] (integer, or float-coded ids as the reference passes them) or features [B, S, d]."""
        cfg = self.cfg
        if x.dim() == 2 and self.embed is not None:
            x = self.embed(x.long())
        if self.attention is not None:
            S, hd = x.shape[1], cfg.input_dim // cfg.num_heads
            if self._rope is None or self._rope[0].shape[0] < S or self._rope[0].device != x.device:
                self._rope = ops.rope_tables(max(S, 128), hd, cfg.rope_base, x.device)
            x = x + self.attention(x, rope=self._rope)
        if self.hss is not None:
            x = self.hss(x)
        aux = x.new_zeros((), dtype=torch.float32)
        if self.ser is not None:
            x = self.ser(x)
            aux = aux + self.ser.aux_loss
        if self.arc is not None:
            x = self.arc(x)
        if self.npe is not None:
            x = self.npe(x.float()).to(x.dtype)
        if self.fm is not None:
            x = self.fm(x)
        self.aux_loss = aux
        return self.head(x) if self.head is not None else x

    def train_step_loss(self, x, target):
        """MSE objective of the reference's C trainer (kernel/train/trainer.c:162-203) plus router auxiliaries."""
        y = self(x)
        return tnn.functional.mse_loss(y.float(), target.float()) + self.aux_loss


SNEPPXModel = Model

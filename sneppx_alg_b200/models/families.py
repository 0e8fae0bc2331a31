"""BERT / GPT / T5 / ViT (the reference's ``model_implementations.py`` and ``vision_transformers.py``): encoder,
decoder, encoder-decoder and vision transformers assembled from this package's layers, so that every projection is
a tcgen05 GEMM and every unbiased self-attention a flash-kernel call on CUDA bf16 tensors."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as tnn
import torch.nn.functional as F

from ..nn.attention import CrossAttention, blockwise_attention
from ..nn.modules import Embedding, LayerNorm, Linear, Module, MultiheadAttention, RMSNorm
from ..ops import functional as ops


class _FFN(Module):
    def __init__(self, d, d_ff, act="gelu", bias=True, dtype=None, device=None):
        super().__init__()
        self.fc1 = Linear(d, d_ff, bias=bias, dtype=dtype, device=device, init_std=0.02)
        self.fc2 = Linear(d_ff, d, bias=bias, dtype=dtype, device=device, init_std=0.02)
        self.act = {"gelu": F.gelu, "relu": F.relu, "silu": F.silu}[act]

    def forward(self, x):
        return self.fc2(self.act(self.fc1(x)))


class _Block(Module):
    """Transformer block; ``pre_ln`` True = GPT/ViT ordering, False = BERT post-LN ordering."""

    def __init__(self, d, heads, d_ff, causal, pre_ln, eps=1e-5, act="gelu", dtype=None, device=None):
        super().__init__()
        self.pre_ln = pre_ln
        self.ln1 = LayerNorm(d, eps=eps, dtype=dtype, device=device)
        self.attn = MultiheadAttention(d, heads, bias=True, causal=causal, dtype=dtype, device=device)
        self.ln2 = LayerNorm(d, eps=eps, dtype=dtype, device=device)
        self.ffn = _FFN(d, d_ff, act, dtype=dtype, device=device)

    def forward(self, x):
        if self.pre_ln:
            x = x + self.attn(self.ln1(x))
            return x + self.ffn(self.ln2(x))
        x = self.ln1(x + self.attn(x))
        return self.ln2(x + self.ffn(x))


# ----------------------------------------------------------------------------- BERT
@dataclass
class BertConfig:
    vocab_size: int = 30522
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    max_position_embeddings: int = 512
    type_vocab_size: int = 2
    layer_norm_eps: float = 1e-12


class BertModel(Module):
    def __init__(self, cfg: BertConfig = None, dtype=None, device=None, **kw):
        super().__init__()
        cfg = cfg or BertConfig(**kw)
        self.config = cfg
        d = cfg.hidden_size
        self.word = Embedding(cfg.vocab_size, d, dtype=dtype, device=device)
        self.pos = Embedding(cfg.max_position_embeddings, d, dtype=dtype, device=device)
        self.type_emb = Embedding(cfg.type_vocab_size, d, dtype=dtype, device=device)
        self.emb_ln = LayerNorm(d, eps=cfg.layer_norm_eps, dtype=dtype, device=device)
        self.layers = tnn.ModuleList([_Block(d, cfg.num_attention_heads, cfg.intermediate_size, False, False,
                                             cfg.layer_norm_eps, dtype=dtype, device=device)
                                      for _ in range(cfg.num_hidden_layers)])
        self.pooler = Linear(d, d, dtype=dtype, device=device, init_std=0.02)

    def forward(self, input_ids, token_type_ids=None):
        B, S = input_ids.shape
        tt = token_type_ids if token_type_ids is not None else torch.zeros_like(input_ids)
        x = self.emb_ln(self.word(input_ids) + self.pos(torch.arange(S, device=input_ids.device))[None] + self.type_emb(tt))
        for layer in self.layers:
            x = layer(x)
        return {"last_hidden_state": x, "pooler_output": torch.tanh(self.pooler(x[:, 0]))}


class BertForMaskedLM(Module):
    def __init__(self, cfg: BertConfig = None, dtype=None, device=None, **kw):
        super().__init__()
        self.bert = BertModel(cfg, dtype, device, **kw)
        d = self.bert.config.hidden_size
        self.transform = Linear(d, d, dtype=dtype, device=device, init_std=0.02)
        self.ln = LayerNorm(d, eps=self.bert.config.layer_norm_eps, dtype=dtype, device=device)
        self.bias = tnn.Parameter(torch.zeros(self.bert.config.vocab_size, dtype=dtype, device=device))

    def forward(self, input_ids, labels=None, token_type_ids=None):
        h = self.ln(F.gelu(self.transform(self.bert(input_ids, token_type_ids)["last_hidden_state"])))
        logits = ops.linear(h, self.bert.word.weight, self.bias)
        out = {"logits": logits}
        if labels is not None:
            out["loss"] = ops.cross_entropy(logits.reshape(-1, logits.shape[-1]), labels.reshape(-1))
        return out


# ----------------------------------------------------------------------------- GPT
@dataclass
class GPTConfig:
    vocab_size: int = 50257
    n_positions: int = 1024
    n_embd: int = 768
    n_layer: int = 12
    n_head: int = 12
    layer_norm_eps: float = 1e-5


class GPTModel(Module):
    """GPT-2 shape: learned positions, pre-LN blocks, tied LM head. ``hidden_states`` is the stack without the head;
    ``forward`` applies the tied head (logits, or the loss when labels are given)."""

    def __init__(self, cfg: GPTConfig = None, dtype=None, device=None, **kw):
        super().__init__()
        cfg = cfg or GPTConfig(**kw)
        self.config = cfg
        d = cfg.n_embd
        self.wte = Embedding(cfg.vocab_size, d, dtype=dtype, device=device)
        self.wpe = Embedding(cfg.n_positions, d, dtype=dtype, device=device)
        self.layers = tnn.ModuleList([_Block(d, cfg.n_head, 4 * d, True, True, cfg.layer_norm_eps, dtype=dtype,
                                             device=device) for _ in range(cfg.n_layer)])
        self.ln_f = LayerNorm(d, eps=cfg.layer_norm_eps, dtype=dtype, device=device)

    def hidden_states(self, input_ids):
        S = input_ids.shape[1]
        x = self.wte(input_ids) + self.wpe(torch.arange(S, device=input_ids.device))[None]
        for layer in self.layers:
            x = layer(x)
        return self.ln_f(x)

    def forward(self, input_ids, labels=None, **_):
        x = self.hidden_states(input_ids)
        if labels is not None:
            loss = ops.linear_cross_entropy(x[:, :-1].reshape(-1, x.shape[-1]), self.wte.weight, labels[:, 1:].reshape(-1))
            return {"loss": loss}
        return {"logits": ops.linear(x, self.wte.weight)}


class GPTLMHeadModel(GPTModel):
    """GPT-2 with an untied output projection of its own (``lm_head``), initialised from the token embedding."""

    def __init__(self, cfg: GPTConfig = None, dtype=None, device=None, **kw):
        super().__init__(cfg, dtype, device, **kw)
        from ..nn.modules import Linear
        self.lm_head = Linear(self.config.n_embd, self.config.vocab_size, bias=False, dtype=dtype, device=device)
        with torch.no_grad():
            self.lm_head.weight.copy_(self.wte.weight)

    def forward(self, input_ids, labels=None, **_):
        x = self.hidden_states(input_ids)
        if labels is not None:
            loss = ops.linear_cross_entropy(x[:, :-1].reshape(-1, x.shape[-1]), self.lm_head.weight, labels[:, 1:].reshape(-1))
            return {"loss": loss}
        return {"logits": ops.linear(x, self.lm_head.weight)}


GPT2LMHeadModel = GPTModel


# ----------------------------------------------------------------------------- T5
@dataclass
class T5Config:
    vocab_size: int = 32128
    d_model: int = 512
    d_ff: int = 2048
    num_layers: int = 6
    num_decoder_layers: int = 6
    num_heads: int = 8
    relative_attention_num_buckets: int = 32
    relative_attention_max_distance: int = 128
    layer_norm_epsilon: float = 1e-6


def t5_relative_bucket(rel, bidirectional, num_buckets, max_distance):
    """T5's log-spaced relative position buckets."""
    ret = torch.zeros_like(rel)
    n = num_buckets
    if bidirectional:
        n //= 2
        ret = ret + (rel > 0).long() * n
        rel = rel.abs()
    else:
        rel = (-rel).clamp_min(0)
    max_exact = n // 2
    large = max_exact + (torch.log(rel.float().clamp_min(1) / max_exact) / math.log(max_distance / max_exact)
                         * (n - max_exact)).long()
    return ret + torch.where(rel < max_exact, rel, large.clamp_max(n - 1))


class _T5SelfAttention(Module):
    def __init__(self, cfg, causal, has_bias_table, dtype=None, device=None):
        super().__init__()
        self.H, self.D, self.causal, self.cfg = cfg.num_heads, cfg.d_model // cfg.num_heads, causal, cfg
        self.qkv = Linear(cfg.d_model, 3 * cfg.d_model, bias=False, dtype=dtype, device=device, init_std=0.02)
        self.o = Linear(cfg.d_model, cfg.d_model, bias=False, dtype=dtype, device=device, init_std=0.02)
        self.rel = Embedding(cfg.relative_attention_num_buckets, cfg.num_heads, dtype=dtype, device=device) \
            if has_bias_table else None

    def bias(self, S, device):
        ctx = torch.arange(S, device=device)
        b = t5_relative_bucket(ctx[None, :] - ctx[:, None], not self.causal, self.cfg.relative_attention_num_buckets,
                               self.cfg.relative_attention_max_distance)
        return self.rel(b).permute(2, 0, 1)[None].float()

    def forward(self, x, bias):
        B, S, d = x.shape
        q, k, v = [t.reshape(B, S, self.H, self.D) for t in self.qkv(x).split(d, dim=-1)]
        o = blockwise_attention(q, k, v, bias=bias, causal=self.causal, scale=1.0)     # T5 does not scale scores
        return self.o(o.reshape(B, S, d))


class _T5Layer(Module):
    def __init__(self, cfg, decoder, first, dtype=None, device=None):
        super().__init__()
        eps = cfg.layer_norm_epsilon
        self.ln1 = RMSNorm(cfg.d_model, eps, dtype=dtype, device=device)
        self.self_attn = _T5SelfAttention(cfg, decoder, first, dtype, device)
        self.cross = CrossAttention(cfg.d_model, cfg.num_heads, dtype=dtype, device=device) if decoder else None
        self.ln_c = RMSNorm(cfg.d_model, eps, dtype=dtype, device=device) if decoder else None
        self.ln2 = RMSNorm(cfg.d_model, eps, dtype=dtype, device=device)
        self.ffn = _FFN(cfg.d_model, cfg.d_ff, "relu", bias=False, dtype=dtype, device=device)

    def forward(self, x, bias, memory=None):
        x = x + self.self_attn(self.ln1(x), bias)
        if self.cross is not None:
            x = x + self.cross(self.ln_c(x), memory)
        return x + self.ffn(self.ln2(x))


class T5ForConditionalGeneration(Module):
    def __init__(self, cfg: T5Config = None, dtype=None, device=None, **kw):
        super().__init__()
        cfg = cfg or T5Config(**kw)
        self.config = cfg
        self.shared = Embedding(cfg.vocab_size, cfg.d_model, dtype=dtype, device=device)
        self.encoder = tnn.ModuleList([_T5Layer(cfg, False, i == 0, dtype, device) for i in range(cfg.num_layers)])
        self.decoder = tnn.ModuleList([_T5Layer(cfg, True, i == 0, dtype, device) for i in range(cfg.num_decoder_layers)])
        self.enc_norm = RMSNorm(cfg.d_model, cfg.layer_norm_epsilon, dtype=dtype, device=device)
        self.dec_norm = RMSNorm(cfg.d_model, cfg.layer_norm_epsilon, dtype=dtype, device=device)

    def encode(self, input_ids):
        x = self.shared(input_ids)
        bias = self.encoder[0].self_attn.bias(x.shape[1], x.device)
        for layer in self.encoder:
            x = layer(x, bias)
        return self.enc_norm(x)

    def decode(self, decoder_input_ids, memory):
        y = self.shared(decoder_input_ids)
        bias = self.decoder[0].self_attn.bias(y.shape[1], y.device)
        for layer in self.decoder:
            y = layer(y, bias, memory)
        return self.dec_norm(y)

    def forward(self, input_ids, decoder_input_ids, labels=None):
        y = self.decode(decoder_input_ids, self.encode(input_ids)) * (self.config.d_model ** -0.5)
        logits = ops.linear(y, self.shared.weight)
        out = {"logits": logits}
        if labels is not None:
            out["loss"] = ops.cross_entropy(logits.reshape(-1, logits.shape[-1]), labels.reshape(-1))
        return out


class T5Model(T5ForConditionalGeneration):
    """Encoder-decoder stack without the output projection: ``forward`` returns the decoder's and the encoder's final
    hidden states (reference: interface_bindings/model_implementations.py:1284)."""

    def forward(self, input_ids, decoder_input_ids):
        mem = self.encode(input_ids)
        return {"last_hidden_state": self.decode(decoder_input_ids, mem), "encoder_last_hidden_state": mem}


# ----------------------------------------------------------------------------- ViT
@dataclass
class ViTConfig:
    image_size: int = 224
    patch_size: int = 16
    num_channels: int = 3
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    num_classes: int = 1000
    layer_norm_eps: float = 1e-6


class VisionTransformer(Module):
    """Patch embedding as one GEMM over unfolded patches, class token, learned positions, pre-LN encoder."""

    def __init__(self, cfg: ViTConfig = None, dtype=None, device=None, **kw):
        super().__init__()
        cfg = cfg or ViTConfig(**kw)
        self.config = cfg
        d, p = cfg.hidden_size, cfg.patch_size
        self.n_patches = (cfg.image_size // p) ** 2
        self.patch = Linear(cfg.num_channels * p * p, d, dtype=dtype, device=device, init_std=0.02)
        self.cls = tnn.Parameter(torch.zeros(1, 1, d, dtype=dtype, device=device))
        self.pos = tnn.Parameter(torch.randn(1, self.n_patches + 1, d, dtype=dtype, device=device) * 0.02)
        self.layers = tnn.ModuleList([_Block(d, cfg.num_attention_heads, cfg.intermediate_size, False, True,
                                             cfg.layer_norm_eps, dtype=dtype, device=device)
                                      for _ in range(cfg.num_hidden_layers)])
        self.ln = LayerNorm(d, eps=cfg.layer_norm_eps, dtype=dtype, device=device)
        self.head = Linear(d, cfg.num_classes, dtype=dtype, device=device, init_std=0.02)

    def patchify(self, img):
        p = self.config.patch_size
        B, C, H, W = img.shape
        x = img.reshape(B, C, H // p, p, W // p, p).permute(0, 2, 4, 1, 3, 5)
        return x.reshape(B, (H // p) * (W // p), C * p * p)

    def forward(self, pixel_values, labels=None):
        x = self.patch(self.patchify(pixel_values))
        x = torch.cat([self.cls.expand(x.shape[0], -1, -1), x], dim=1) + self.pos
        for layer in self.layers:
            x = layer(x)
        logits = self.head(self.ln(x)[:, 0])
        out = {"logits": logits}
        if labels is not None:
            out["loss"] = F.cross_entropy(logits.float(), labels)
        return out


ViTForImageClassification = VisionTransformer


# ----------------------------------------------------------------------------- masked autoencoder
class MAE(Module):
    """Masked autoencoder for images (He et al. 2021; reference: interface_bindings/vision_transformers.py:651).

    A random ``mask_ratio`` of the patches is dropped; the encoder sees only the kept ones (plus a class token), a
    lighter decoder gets the encoded tokens back in place with a learned mask token everywhere else and predicts the
    pixels of every patch; the loss is the mean squared error on the dropped patches only.
    ``forward(imgs)`` returns ``(loss, pred, mask)`` with pred [B, N, p*p*C] and mask [B, N] (1 = dropped)."""

    def __init__(self, img_size=224, patch_size=16, in_channels=3, embed_dim=768, encoder_depth=12, decoder_depth=8,
                 num_heads=12, mlp_ratio=4.0, mask_ratio=0.75, decoder_embed_dim=512, decoder_num_heads=None,
                 norm_pix_loss=False, dtype=None, device=None):
        super().__init__()
        assert img_size % patch_size == 0
        self.patch_size, self.in_channels, self.mask_ratio, self.norm_pix_loss = patch_size, in_channels, mask_ratio, norm_pix_loss
        self.n_patches = n = (img_size // patch_size) ** 2
        pd = in_channels * patch_size * patch_size
        kw = dict(dtype=dtype, device=device)
        self.patch = Linear(pd, embed_dim, init_std=0.02, **kw)
        self.cls = tnn.Parameter(torch.zeros(1, 1, embed_dim, **kw))
        self.pos = tnn.Parameter(torch.randn(1, n + 1, embed_dim, **kw) * 0.02)
        self.encoder = tnn.ModuleList([_Block(embed_dim, num_heads, int(embed_dim * mlp_ratio), False, True, **kw)
                                       for _ in range(encoder_depth)])
        self.enc_norm = LayerNorm(embed_dim, **kw)
        self.to_decoder = Linear(embed_dim, decoder_embed_dim, init_std=0.02, **kw)
        self.mask_token = tnn.Parameter(torch.randn(1, 1, decoder_embed_dim, **kw) * 0.02)
        self.dec_pos = tnn.Parameter(torch.randn(1, n + 1, decoder_embed_dim, **kw) * 0.02)
        dh = decoder_num_heads or max(1, min(num_heads, decoder_embed_dim // 32))
        self.decoder = tnn.ModuleList([_Block(decoder_embed_dim, dh, int(decoder_embed_dim * mlp_ratio), False, True, **kw)
                                       for _ in range(decoder_depth)])
        self.dec_norm = LayerNorm(decoder_embed_dim, **kw)
        self.to_pixels = Linear(decoder_embed_dim, pd, init_std=0.02, **kw)

    def patchify(self, img):
        p = self.patch_size
        B, C, H, W = img.shape
        x = img.reshape(B, C, H // p, p, W // p, p).permute(0, 2, 4, 1, 3, 5)
        return x.reshape(B, (H // p) * (W // p), C * p * p)

    def unpatchify(self, patches):
        p, C = self.patch_size, self.in_channels
        B, N, _ = patches.shape
        g = int(N ** 0.5)
        x = patches.reshape(B, g, g, C, p, p).permute(0, 3, 1, 4, 2, 5)
        return x.reshape(B, C, g * p, g * p)

    def random_masking(self, x, mask_ratio=None, noise=None):
        """Keeps the ``1 - mask_ratio`` patches with the smallest noise. Returns (kept tokens, mask [B, N] with 1 for
        dropped, restore indices that undo the shuffle)."""
        B, N, D = x.shape
        ratio = self.mask_ratio if mask_ratio is None else mask_ratio
        keep = max(1, int(round(N * (1.0 - ratio))))
        noise = torch.rand(B, N, device=x.device) if noise is None else noise
        shuffle = noise.argsort(dim=1)
        restore = shuffle.argsort(dim=1)
        kept = x.gather(1, shuffle[:, :keep, None].expand(-1, -1, D))
        mask = torch.ones(B, N, device=x.device)
        mask[:, :keep] = 0
        return kept, mask.gather(1, restore), restore

    def encode(self, imgs, mask_ratio=None, noise=None):
        x = self.patch(self.patchify(imgs).to(self.patch.weight.dtype)) + self.pos[:, 1:]
        x, mask, restore = self.random_masking(x, mask_ratio, noise)
        x = torch.cat([(self.cls + self.pos[:, :1]).expand(x.shape[0], -1, -1), x], dim=1)
        for layer in self.encoder:
            x = layer(x)
        return self.enc_norm(x), mask, restore

    def decode(self, latent, restore):
        x = self.to_decoder(latent)
        B, _, D = x.shape
        N = restore.shape[1]
        filled = torch.cat([x[:, 1:], self.mask_token.expand(B, N + 1 - x.shape[1], -1).to(x.dtype)], dim=1)
        filled = filled.gather(1, restore[:, :, None].expand(-1, -1, D))
        x = torch.cat([x[:, :1], filled], dim=1) + self.dec_pos
        for layer in self.decoder:
            x = layer(x)
        return self.to_pixels(self.dec_norm(x))[:, 1:]

    def reconstruction_loss(self, imgs, pred, mask):
        target = self.patchify(imgs).float()
        if self.norm_pix_loss:
            target = (target - target.mean(-1, keepdim=True)) / (target.var(-1, keepdim=True) + 1e-6).sqrt()
        per_patch = (pred.float() - target).pow(2).mean(-1)
        return (per_patch * mask).sum() / mask.sum().clamp_min(1.0)

    def forward(self, imgs, mask_ratio=None, noise=None):
        latent, mask, restore = self.encode(imgs, mask_ratio, noise)
        pred = self.decode(latent, restore)
        return self.reconstruction_loss(imgs, pred, mask), pred, mask


def mae_base(**kw) -> MAE:
    return MAE(**{**dict(embed_dim=768, encoder_depth=12, num_heads=12, decoder_embed_dim=512, decoder_depth=8), **kw})


def mae_large(**kw) -> MAE:
    return MAE(**{**dict(embed_dim=1024, encoder_depth=24, num_heads=16, decoder_embed_dim=512, decoder_depth=8), **kw})

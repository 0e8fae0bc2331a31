"""Attention variants against dense fp32 references (reference tests: tests/unit/test_flash_attention.c,
test_flex_attention.c, test_alibi.c)."""
import math

import torch

from sneppx_alg_b200.nn import attention as A
from sneppx_alg_b200.ops import functional as F


def _dense(q, k, v, bias=None, keep=None, scale=None):
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * (scale or 1 / math.sqrt(q.shape[-1]))
    if bias is not None:
        s = s + bias
    if keep is not None:
        s = s.masked_fill(~keep, -float("inf"))
    return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), v.float())


def test_blockwise_matches_dense_with_bias_mask_and_block_skip():
    torch.manual_seed(0)
    B, S, H, D = 2, 70, 4, 16
    q, k, v = torch.randn(B, S, H, D), torch.randn(B, S, H, D), torch.randn(B, S, H, D)
    bias = A.alibi_bias(H, S, S)[None]
    causal = torch.tril(torch.ones(S, S, dtype=torch.bool))
    o = A.blockwise_attention(q, k, v, bias=bias, causal=True, block=32)
    assert torch.allclose(o, _dense(q, k, v, bias, causal), atol=1e-5)
    fn = lambda qi, kj: (kj <= qi) & ((qi - kj < 8) | (kj % 16 == 0))  # noqa: E731
    bm, full = A.FlexAttention.create_block_mask(fn, S, S, 32)
    o = A.blockwise_attention(q, k, v, mask=full, block_mask=bm, block=32)
    assert torch.allclose(o, _dense(q, k, v, None, full), atol=1e-5)
    # score_mod: soft-capping
    o = A.blockwise_attention(q, k, v, score_mod=lambda s, b, h, qi, kj: 5 * torch.tanh(s / 5), block=16)
    s = torch.einsum("bqhd,bkhd->bhqk", q, k) / math.sqrt(D)
    ref = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(5 * torch.tanh(s / 5), -1), v)
    assert torch.allclose(o, ref, atol=1e-5)
    # GQA + different key length (cross attention)
    k2, v2 = torch.randn(B, 33, 2, D), torch.randn(B, 33, 2, D)
    o = A.blockwise_attention(q, k2, v2, block=16)
    assert torch.allclose(o, _dense(q, k2.repeat_interleave(2, 2), v2.repeat_interleave(2, 2)), atol=1e-5)


def test_alibi_slopes():
    s8 = A.alibi_slopes(8)
    assert torch.allclose(s8, torch.tensor([2.0 ** -(i + 1) for i in range(8)]))
    assert A.alibi_slopes(12).shape == (12,)


def test_modules_forward_backward():
    torch.manual_seed(0)
    x = torch.randn(2, 24, 64)
    mods = [A.Attention(64, 4, 2), A.SlidingWindowAttention(64, 4, window=8), A.DifferentialAttention(64, 4),
            A.FlexAttention(64, 4, block_size=8), A.SparseAttention(64, 4, local=4, stride=8, block_size=8),
            A.ALiBiAttention(64, 4, block_size=8), A.MultiHeadLatentAttention(64, 4, 16, 8, 16, 8, 16),
            A.MixtureOfDepths(64, torch.nn.Linear(64, 64), 0.5)]
    for m in mods:
        y = m(x)
        assert y.shape == x.shape and torch.isfinite(y).all(), type(m).__name__
        y.sum().backward()
    ca = A.CrossAttention(64, 4, d_context=32)
    assert ca(x, torch.randn(2, 7, 32)).shape == x.shape


def test_kv_cache_decode_matches_full():
    torch.manual_seed(0)
    m = A.Attention(32, 4)
    x = torch.randn(1, 10, 32)
    full = m(x)
    cache = {}
    m(x[:, :9], kv_cache=cache)
    last = m(x[:, 9:], kv_cache=cache, start_pos=9)
    assert torch.allclose(last[:, 0], full[:, 9], atol=1e-5)
    mla = A.MultiHeadLatentAttention(32, 2, 8, 0, 8, 4, 8)
    full = mla(x)
    c = {}
    mla(x[:, :9], latent_cache=c)
    last = mla(x[:, 9:], latent_cache=c)
    assert c["latent"].shape == (1, 10, 12) and torch.allclose(last[:, 0], full[:, 9], atol=1e-5)


def test_sliding_window_reference():
    torch.manual_seed(0)
    q, k, v = torch.randn(1, 20, 2, 8), torch.randn(1, 20, 2, 8), torch.randn(1, 20, 2, 8)
    i, j = torch.arange(20)[:, None], torch.arange(20)[None]
    keep = (j <= i) & (i - j < 5)
    assert torch.allclose(F.attention(q, k, v, causal=True, window=5), _dense(q, k, v, None, keep), atol=1e-5)

"""BERT / GPT / T5 / ViT and the small reference models: shapes, losses fall, T5 buckets match the published rule."""
import torch

from sneppx_alg_b200.models import families as M
from sneppx_alg_b200.models import small as S


def _fit(model, loss_fn, steps=25, lr=3e-3):
    opt = torch.optim.Adam(model.parameters(), lr)
    first = last = None
    for _ in range(steps):
        loss = loss_fn()
        opt.zero_grad()
        loss.backward()
        opt.step()
        last = loss.item()
        first = first if first is not None else last
    return first, last


def test_bert_gpt_t5_vit():
    torch.manual_seed(0)
    ids = torch.randint(0, 100, (2, 12))
    bert = M.BertForMaskedLM(vocab_size=100, hidden_size=32, num_hidden_layers=2, num_attention_heads=4,
                             intermediate_size=64, max_position_embeddings=16)
    out = bert(ids, labels=ids)
    assert out["logits"].shape == (2, 12, 100)
    a, b = _fit(bert, lambda: bert(ids, labels=ids)["loss"])
    assert b < a
    gpt = M.GPTModel(vocab_size=100, n_positions=16, n_embd=32, n_layer=2, n_head=4)
    assert gpt(ids)["logits"].shape == (2, 12, 100)
    a, b = _fit(gpt, lambda: gpt(ids, labels=ids)["loss"])
    assert b < a
    # causality: changing a later token leaves earlier logits unchanged
    ids2 = ids.clone()
    ids2[:, -1] = (ids2[:, -1] + 1) % 100
    assert torch.allclose(gpt(ids)["logits"][:, :-1], gpt(ids2)["logits"][:, :-1], atol=1e-5)
    t5 = M.T5ForConditionalGeneration(vocab_size=100, d_model=32, d_ff=64, num_layers=2, num_decoder_layers=2, num_heads=4)
    out = t5(ids, ids[:, :7], labels=ids[:, :7])
    assert out["logits"].shape == (2, 7, 100) and torch.isfinite(out["loss"])
    out["loss"].backward()
    vit = M.VisionTransformer(image_size=32, patch_size=8, hidden_size=32, num_hidden_layers=2, num_attention_heads=4,
                              intermediate_size=64, num_classes=10)
    img = torch.randn(3, 3, 32, 32)
    out = vit(img, labels=torch.tensor([1, 2, 3]))
    assert out["logits"].shape == (3, 10)
    # patchify is an exact rearrangement
    p = vit.patchify(img)
    assert torch.equal(p[0, 0].view(3, 8, 8), img[0, :, :8, :8]) and torch.equal(p[0, 5].view(3, 8, 8), img[0, :, 8:16, 8:16])


def test_t5_bucket_rule():
    rel = torch.arange(-10, 11)[None]
    b = M.t5_relative_bucket(rel, True, 32, 128)
    assert b.min() >= 0 and b.max() < 32 and b[0, 10] == 0 and b[0, 11] == 17 and b[0, 9] == 1
    c = M.t5_relative_bucket(rel, False, 32, 128)
    assert (c[0, 10:] == 0).all() and c[0, 9] == 1


def test_small_models():
    torch.manual_seed(0)
    adj = (torch.rand(10, 10) > 0.6).float()
    adj = ((adj + adj.T) > 0).float()
    gcn = S.GCN(8, 16, 3)
    x, y = torch.randn(10, 8), torch.randint(0, 3, (10,))
    a, b = _fit(gcn, lambda: torch.nn.functional.cross_entropy(gcn(x, adj), y))
    assert b < a
    an = S.GCNLayer.normalize(adj)
    assert torch.allclose(an, an.T, atol=1e-6)
    for cell in ("rnn", "gru", "lstm"):
        rnn = S.RNN(4, 8, cell)
        out, (h, c) = rnn(torch.randn(2, 5, 4))
        assert out.shape == (2, 5, 8) and torch.equal(out[:, -1], h)
    lstm = S.RNN(4, 8, "lstm")
    ref = torch.nn.LSTM(4, 8, batch_first=True)
    with torch.no_grad():
        ref.weight_ih_l0.copy_(lstm.wx.weight)
        ref.weight_hh_l0.copy_(lstm.wh.weight)
        ref.bias_ih_l0.copy_(lstm.wx.bias)
        ref.bias_hh_l0.zero_()
    xx = torch.randn(2, 6, 4)
    assert torch.allclose(lstm(xx)[0], ref(xx)[0], atol=1e-5)
    gan = S.GAN(8, 16, 32)
    real = torch.randn(4, 16).tanh()
    assert torch.isfinite(gan.discriminator_loss(real)) and torch.isfinite(gan.generator_loss(4))
    diff = S.Diffusion(6, 32, steps=50)
    data = torch.randn(64, 6) * 0.1 + 1.0
    a, b = _fit(diff, lambda: diff.loss(data), steps=40)
    assert b < a and diff.sample(3, 6, steps=5).shape == (3, 6)
    agent = S.PolicyGradientAgent(4, 2)
    acts, lps, vals = agent.act(torch.randn(5, 4))
    loss = agent.loss(lps, vals, [1.0, 0.0, 1.0, 1.0, 0.0])
    loss.backward()
    assert torch.allclose(agent.returns([1.0, 1.0]), torch.tensor([1.99, 1.0]))

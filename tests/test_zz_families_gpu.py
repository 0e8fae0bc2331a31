"""Model families other than the causal language models, in bf16 on the GPU (linear layers, LayerNorm and attention
go through this package's kernels): the loss of a forward pass equals the fp32 CPU loss of the same weights within
bf16 tolerance, and backward leaves finite gradients on every parameter."""
import copy

import pytest
import torch

from sneppx_alg_b200.models import families as F
from sneppx_alg_b200.ops import check_status

pytestmark = pytest.mark.gpu

IDS = torch.randint(0, 500, (2, 24), generator=torch.Generator().manual_seed(0))
DEC = torch.randint(0, 500, (2, 9), generator=torch.Generator().manual_seed(1))
IMG = torch.randn(2, 3, 32, 32, generator=torch.Generator().manual_seed(2))
LAB = torch.tensor([1, 3])
NOISE = torch.rand(2, 16, generator=torch.Generator().manual_seed(3))

CASES = {
    "gpt2": (lambda: F.GPTModel(vocab_size=512, n_positions=64, n_embd=256, n_layer=2, n_head=2),
             lambda m, d: m(IDS.to(d), labels=IDS.to(d))["loss"]),
    "gpt_lm_head": (lambda: F.GPTLMHeadModel(vocab_size=512, n_positions=64, n_embd=256, n_layer=1, n_head=2),
                    lambda m, d: m(IDS.to(d), labels=IDS.to(d))["loss"]),
    "bert_mlm": (lambda: F.BertForMaskedLM(vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=2,
                                           intermediate_size=512, max_position_embeddings=64),
                 lambda m, d: m(IDS.to(d), labels=IDS.to(d))["loss"]),
    "vit": (lambda: F.VisionTransformer(image_size=32, patch_size=8, num_channels=3, hidden_size=256, num_hidden_layers=2,
                                        num_attention_heads=2, intermediate_size=512, num_classes=10),
            lambda m, d: m(IMG.to(d, dtype=next(m.parameters()).dtype), labels=LAB.to(d))["loss"]),
    "mae": (lambda: F.MAE(img_size=32, patch_size=8, embed_dim=256, encoder_depth=2, decoder_depth=1, num_heads=2,
                          decoder_embed_dim=128, decoder_num_heads=1),
            lambda m, d: m(IMG.to(d, dtype=next(m.parameters()).dtype), noise=NOISE.to(d))[0]),
    "t5": (lambda: F.T5ForConditionalGeneration(vocab_size=512, d_model=256, d_ff=512, num_layers=1, num_decoder_layers=1, num_heads=2),
           lambda m, d: m(IDS.to(d), DEC.to(d), labels=DEC.to(d))["loss"]),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_family_bf16_matches_fp32_reference(name):
    build, loss_of = CASES[name]
    torch.manual_seed(0)
    ref = build().float()
    gpu = copy.deepcopy(ref).to(device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        want = float(loss_of(ref, "cpu"))
    got = loss_of(gpu, "cuda")
    got.backward()
    torch.cuda.synchronize()
    check_status()
    got = float(got.detach())
    assert abs(got - want) < 0.03 * max(1.0, abs(want)), (name, got, want)
    grads = [p.grad for p in gpu.parameters() if p.grad is not None]
    assert len(grads) >= 10 and all(torch.isfinite(g.float()).all().item() for g in grads)

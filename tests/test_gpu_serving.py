"""Serving kernels on the GPU: KV append + RoPE, paged decode attention, dequant-GEMM, and the paged engine
end to end against plain cached generation."""
import pytest
import torch

from sneppx_alg_b200 import ops
from sneppx_alg_b200.ops import paged, quant
from sneppx_alg_b200.ops.functional import rope_tables

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)


def test_kv_append_and_paged_decode():
    torch.manual_seed(0)
    B, Hq, Hkv, D, bs, nblk = 5, 8, 2, 128, 16, 64
    kc = torch.zeros(nblk, bs, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    cos, sin = rope_tables(2048, D, 5e5, "cuda")
    lens = [700, 33, 1, 256, 1500]
    tables = torch.zeros(B, 100, dtype=torch.int32)
    free = list(range(nblk * 0, nblk))
    import random
    random.Random(0).shuffle(free)
    need = sum((n + bs - 1) // bs for n in lens)
    kc = torch.zeros(need + 4, bs, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    nxt = 0
    for b, n in enumerate(lens):
        nb = (n + bs - 1) // bs
        tables[b, :nb] = torch.arange(nxt, nxt + nb, dtype=torch.int32)
        nxt += nb
        qkv = torch.randn(n, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
        pos = torch.arange(n, device="cuda", dtype=torch.int32)
        slot = (tables[b, :nb].cuda().repeat_interleave(bs)[:n] * bs + pos % bs).to(torch.int32)
        ref_in = qkv.clone()
        paged.kv_append_(qkv, cos, sin, pos, slot, kc, vc, Hq, Hkv, D)
        ref_f, kc_ref_f, vc_ref_f = ref_in.float(), kc_ref.float(), vc_ref.float()
        paged.kv_append_reference(ref_f, cos, sin, pos, slot, kc_ref_f, vc_ref_f, Hq, Hkv, D)
        kc_ref.copy_(kc_ref_f)
        vc_ref.copy_(vc_ref_f)
        assert _rel(qkv, ref_f) < 1e-2
    assert _rel(kc, kc_ref) < 1e-2 and _rel(vc, vc_ref) < 1e-2
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
    sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    out = paged.paged_decode(q, kc, vc, tables.cuda(), sl)
    ref = paged.paged_decode_reference(q.float(), kc.float(), vc.float(), tables.cuda(), sl)
    assert _rel(out, ref) < 2e-2


@pytest.mark.parametrize("Hq,Hkv,bs", [(32, 8, 16), (8, 8, 16), (16, 2, 32), (12, 4, 8), (8, 2, 128)])
def test_paged_decode_tensor_core(Hq, Hkv, bs, monkeypatch):
    """Tensor-core decode kernel against the fp32 reference and against the SIMT kernel; cache rows that belong to no
    sequence hold NaN, so any read past a sequence's end that reaches the output fails the test."""
    import random
    torch.manual_seed(1)
    D = 128
    lens = [1, 15, 128, 129, 700, 2304, 0, 1000]
    B = len(lens)
    need = sum((n + bs - 1) // bs for n in lens)
    kc = torch.full((need + 3, bs, Hkv, D), float("nan"), device="cuda", dtype=torch.bfloat16)
    vc = torch.full_like(kc, float("nan"))
    order = list(range(need + 3))
    random.Random(3).shuffle(order)
    width = max((n + bs - 1) // bs for n in lens) + 2
    tables = torch.zeros(B, width, dtype=torch.int32)
    nxt = 0
    for b, n in enumerate(lens):
        nb = (n + bs - 1) // bs
        blocks = order[nxt: nxt + nb]
        nxt += nb
        tables[b, :nb] = torch.tensor(blocks, dtype=torch.int32)
        if n:
            k = torch.randn(n, Hkv, D, device="cuda", dtype=torch.bfloat16)
            v = torch.randn(n, Hkv, D, device="cuda", dtype=torch.bfloat16)
            idx = torch.tensor(blocks, device="cuda").repeat_interleave(bs)[:n] * bs + torch.arange(n, device="cuda") % bs
            kc.view(-1, Hkv, D)[idx] = k
            vc.view(-1, Hkv, D)[idx] = v
    q = (torch.randn(B, Hq, D, device="cuda") * 1.5).to(torch.bfloat16)
    sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    assert paged._use_tc(D, bs, Hq // Hkv)
    out = paged.paged_decode(q, kc, vc, tables.cuda(), sl)
    ops.check_status()
    ref = paged.paged_decode_reference(q.float(), kc.float(), vc.float(), tables.cuda(), sl)
    assert torch.isfinite(out.float()).all()
    assert _rel(out, ref) < 2e-2
    monkeypatch.setenv("SX_PAGED_TC", "0")
    simt = paged.paged_decode(q, kc, vc, tables.cuda(), sl)
    assert _rel(out, simt) < 2e-2


@pytest.mark.parametrize("mode", ["fp8", "int4"])
@pytest.mark.parametrize("M,N,K", [(64, 512, 1024), (300, 1000, 256), (2048, 4096, 4096)])
def test_dequant_gemm(mode, M, N, K):
    torch.manual_seed(0)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    if mode == "fp8":
        q, s = quant.quant_fp8_128x128(w)
        wd = quant.dequant_fp8(q, s, "128x128")
        q = q.view(torch.uint8)
    else:
        q, s = quant.quant_int4(w)
        wd = quant.dequant_int4(q, s)
    bias = torch.randn(N, device="cuda")
    y = quant.gemm_dequant(x, q, s, mode, bias)
    ops.check_status()
    ref = x.float() @ wd.float().t() + bias
    assert _rel(y, ref) < 1.5e-2


def test_paged_engine_matches_cached_generation_gpu():
    from sneppx_alg_b200.models import ModelConfig, build_model
    from sneppx_alg_b200.serving.generation import generate
    from sneppx_alg_b200.serving.llm_engine import LLMEngine, SamplingParams
    torch.manual_seed(0)
    cfg = ModelConfig(hidden_size=256, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1,
                      intermediate_size=512, vocab_size=512, max_position_embeddings=512, rms_norm_eps=1e-5)
    model = build_model(cfg, dtype=torch.bfloat16, device="cuda").eval()
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (37, 130, 64, 5)]
    eng = LLMEngine(model, num_blocks=256, block_size=16, max_batch_size=4)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=12))
    ops.check_status()
    agree = 0
    for p, o in zip(prompts, outs):
        ref = generate(model, torch.tensor([p], device="cuda"), max_new_tokens=12)[0, len(p):].tolist()
        agree += sum(int(a == b) for a, b in zip(o, ref))
        assert o[0] == ref[0]            # first token comes from the same prefill math
    assert agree >= 0.7 * 12 * len(prompts)   # bf16 paths differ in reduction order; most greedy tokens coincide
    # weight-only fp8 serving runs end to end
    quant.quantize_model_(model, "fp8")
    eng2 = LLMEngine(model, num_blocks=256, block_size=16)
    assert len(eng2.generate(prompts[:2], SamplingParams(max_new_tokens=4))[0]) == 4
    ops.check_status()

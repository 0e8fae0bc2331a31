"""Model card record, weight collection (dtype conversion, int8 / int4, formats, memory-mapped load) and GGUF files."""
import os
import struct

import pytest
import torch

from sneppx_alg_b200.hub.model_card import ModelCard, WeightCollection, dtype_size, load_gguf, save_gguf


def test_model_card_round_trip_validation_and_markdown(tmp_path):
    card = ModelCard(name="tiny-llama", version="1.2.0", architecture="LlamaForCausalLM", model_type="causal-lm",
                     num_parameters=1_100_000, precision="bf16", license="apache-2.0", intended_use="tests", accuracy=0.5)
    card.add_tag("llm"); card.add_tag("llm"); card.add_tag("tiny")
    assert card.tags == ["llm", "tiny"] and card.validate() == (True, [])
    p = str(tmp_path / "card.json")
    card.save(p)
    assert ModelCard.load(p) == card
    assert ModelCard.from_json(card.to_json(pretty=False)) == card
    md = card.to_markdown()
    assert md.startswith("# tiny-llama 1.2.0") and "| Parameters | 1,100,000 |" in md and "## Intended use" in md and "Tags: llm, tiny" in md
    ok, errors = ModelCard(name="x", precision="fp3", accuracy=2.0, num_layers=-1).validate()
    assert not ok and len(errors) == 5
    with pytest.raises(ValueError):
        ModelCard.from_json('{"num_layers": "many"}')
    with pytest.raises(ValueError):
        ModelCard.from_json("[1, 2]")
    assert ModelCard.from_json('{"name": "a", "future_field": 1, "learning_rate": 1}').learning_rate == 1.0

    from sneppx_alg_b200.models import create_model
    model = create_model("llama3-tiny")
    auto = ModelCard.from_model(model, "auto", license="mit")
    assert auto.validate()[0] and auto.num_parameters == sum(p.numel() for p in model.parameters())
    assert auto.num_layers > 0 and auto.hidden_size > 0 and auto.vocab_size > 0 and auto.license == "mit"


def test_gguf_round_trip_and_damage(tmp_path):
    torch.manual_seed(0)
    tensors = {"tok_embd.weight": torch.randn(64, 32), "blk.0.attn.weight": torch.randn(32, 64).half(),
               "blk.0.norm.weight": torch.randn(32).bfloat16(), "scalar": torch.tensor(3.0)}
    meta = {"general.architecture": "llama", "llama.block_count": 1, "llama.rope.freq_base": 10000.0, "flag": True,
            "tokens": ["a", "b", "c"], "offset": -5}
    p = str(tmp_path / "m.gguf")
    save_gguf(p, tensors, meta)
    back, m = load_gguf(p)
    assert set(back) == set(tensors) and all(torch.equal(back[k], tensors[k]) and back[k].dtype == tensors[k].dtype for k in tensors)
    assert m["general.architecture"] == "llama" and m["llama.block_count"] == 1 and m["tokens"] == ["a", "b", "c"]
    assert m["flag"] is True and m["offset"] == -5 and m["general.alignment"] == 32
    raw = open(p, "rb").read()
    assert raw[:4] == b"GGUF" and struct.unpack_from("<I", raw, 4)[0] == 3

    save_gguf(p, {"w": tensors["tok_embd.weight"]}, q8_0=True)                    # 8-bit blocks: 34 bytes per 32 values
    q, _ = load_gguf(p)
    assert os.path.getsize(p) < 64 * 32 * 4 * 0.4 and (q["w"] - tensors["tok_embd.weight"]).abs().max() < 0.03

    for cut in (3, 10, 40, len(raw) - 40):
        open(p, "wb").write(raw[:cut])
        with pytest.raises(ValueError):
            load_gguf(p)
    open(p, "wb").write(raw[:8] + struct.pack("<Q", 1 << 40) + raw[16:])
    with pytest.raises(ValueError):
        load_gguf(p)


def test_weight_collection_quantisation_and_formats(tmp_path):
    torch.manual_seed(1)
    wc = WeightCollection()
    wc.add("layer.weight", torch.randn(16, 256))
    wc.add("layer.bias", torch.randn(16))
    wc.add("head.weight", torch.randn(8, 128))
    wc.metadata["arch"] = "toy"
    assert wc.names() == ["layer.weight", "layer.bias", "head.weight"] and len(wc) == 3
    ref = {k: v.clone() for k, v in wc.state_dict().items()}
    full = wc.nbytes()
    wc.quantize_int8("layer.weight")
    wc.quantize_int4("head.weight", group=64)
    assert wc.get("layer.weight", dequantize=False).dtype == torch.int8 and wc.nbytes() < 0.5 * full
    assert (wc.get("layer.weight") - ref["layer.weight"]).abs().max() < 0.03
    assert (wc.get("head.weight") - ref["head.weight"]).abs().max() < 0.35 and wc.get("head.weight").shape == (8, 128)
    with pytest.raises(ValueError):
        wc.quantize_int4("layer.bias")
    wc.convert_dtype("bf16")
    assert wc.get("layer.bias").dtype == torch.bfloat16 and wc.get("layer.weight", dequantize=False).dtype == torch.int8
    assert dtype_size("bf16") == 2 and dtype_size("fp32") == 4 and dtype_size("int8") == 1
    assert wc.remove("layer.bias") and not wc.remove("layer.bias")

    plain = WeightCollection()
    for k, v in ref.items():
        plain.add(k, v)
    for ext in (".safetensors", ".gguf", ".npz", ".pth", ".sxh5"):
        p = str(tmp_path / ("w" + ext))
        plain.save(p)
        back = WeightCollection.load(p)
        assert set(back.names()) == set(ref) and all(torch.equal(back.get(k).float(), ref[k]) for k in ref), ext
    mapped = WeightCollection.load(str(tmp_path / "w.safetensors"), mmap=True)
    assert all(torch.equal(mapped.get(k), ref[k]) for k in ref)
    with pytest.raises(ValueError):
        WeightCollection.load(str(tmp_path / "w.bin"))

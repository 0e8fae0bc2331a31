"""Hub / zoo: presets, HF name mapping and conversion order, save / load round trips in every weight format."""
import torch

from sneppx_alg_b200.checkpoint.sneppx_format import load_tensors
from sneppx_alg_b200.hub import (Hub, ModelHub, convert_hf_to_sneppx, from_pretrained, load_hub_container,
                                 load_safetensors, map_hf_name, save_hub_container, save_safetensors)
from sneppx_alg_b200.models import ModelConfig, build_model, config_from_name, extend_context, get_model_config


def test_presets_match_reference_registry():
    c = get_model_config("llama3", "8B")
    assert (c["hidden_size"], c["intermediate_size"], c["num_hidden_layers"], c["num_key_value_heads"], c["vocab_size"],
            c["rope_theta"]) == (4096, 14336, 32, 8, 128256, 5e5)
    assert get_model_config("mistral", "7B")["sliding_window"] == 4096
    assert get_model_config("deepseek_v2", "lite")["kv_lora_rank"] == 512
    info = from_pretrained("meta-llama/Llama-3-8B")
    assert 7.9e9 < info["num_parameters"] < 8.1e9
    assert abs(config_from_name("mamba2-2.7b").estimate_parameters() / 2.7e9 - 1) < 0.15   # ngroups 8 adds B/C projections
    ext = extend_context(config_from_name("llama3-8b"), 131072, "ntk")
    assert ext.max_position_embeddings == 131072 and ext.rope_scale_factor == 16.0


def test_hf_mapping_and_conversion(tmp_path):
    assert map_hf_name("model.layers.3.self_attn.k_proj.weight") == "layers.3.attn.k_proj.weight"
    assert map_hf_name("model.layers.0.post_attention_layernorm.weight") == "layers.0.mlp_norm.weight"
    assert map_hf_name("model.embed_tokens.weight") == "embedding" and map_hf_name("something.else") is None
    cfg = ModelConfig(hidden_size=16, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1,
                      intermediate_size=32, vocab_size=40, max_position_embeddings=16)
    torch.manual_seed(0)
    model = build_model(cfg)
    ref = model.to_reference_state_dict()
    hf = {"model.embed_tokens.weight": ref["embedding"], "model.norm.weight": ref["norm"], "lm_head.weight": ref["lm_head"]}
    for i in range(2):
        p, q = f"layers.{i}.", f"model.layers.{i}."
        hf[q + "input_layernorm.weight"] = ref[p + "attn_norm.weight"]
        hf[q + "post_attention_layernorm.weight"] = ref[p + "mlp_norm.weight"]
        for x in "qkvo":
            hf[q + f"self_attn.{x}_proj.weight"] = ref[p + f"attn.{x}_proj.weight"]
        for x in ("gate", "up", "down"):
            hf[q + f"mlp.{x}_proj.weight"] = ref[p + f"mlp.{x}_proj.weight"]
    order = convert_hf_to_sneppx(hf, str(tmp_path / "m.sneppx"), cfg)
    assert order[:4] == ["embedding", "norm", "lm_head", "layers.0.attn_norm.weight"] and len(order) == 3 + 2 * 9
    tensors, meta = load_tensors(str(tmp_path / "m.sneppx"))
    assert meta["family"] == "llama" and meta["num_converted"] == 21
    other = build_model(cfg)
    other.load_reference_state_dict(tensors)
    ids = torch.randint(0, 40, (1, 8))
    assert torch.allclose(other(ids)["logits"], model(ids)["logits"], atol=1e-5)


def test_save_pretrained_formats_and_hub(tmp_path):
    cfg = ModelConfig(hidden_size=16, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=2,
                      intermediate_size=32, vocab_size=40, max_position_embeddings=16)
    model = build_model(cfg)
    ids = torch.randint(0, 40, (1, 8))
    for fmt in ("sneppx", "safetensors"):
        d = ModelHub.save_pretrained(model, str(tmp_path / fmt), fmt)
        back = from_pretrained(d)
        assert torch.allclose(back(ids)["logits"], model(ids)["logits"], atol=1e-5)
    hub = Hub(str(tmp_path / "hub"))
    hub.upload(str(tmp_path / "sneppx"), "org/tiny", "1.0.0", tags=["llama"], metrics={"ppl": 12.0})
    hub.upload(str(tmp_path / "sneppx"), "org/tiny", "1.1.0", tags=["llama"], metrics={"ppl": 11.0})
    assert hub.list_models() == {"org/tiny": ["1.0.0", "1.1.0"]} and hub.search("tiny", tag="llama") == ["org/tiny"]
    assert hub.leaderboard("ppl", higher_is_better=False)[0][1] == "1.1.0"
    assert torch.allclose(hub.load("org/tiny")(ids)["logits"], model(ids)["logits"], atol=1e-5)
    t = {"a": torch.randn(3, 4), "b": torch.arange(5, dtype=torch.int64)}
    save_hub_container(str(tmp_path / "c.bin"), t, {"k": 1})
    back, meta = load_hub_container(str(tmp_path / "c.bin"))
    assert meta["k"] == 1 and torch.equal(back["a"], t["a"]) and torch.equal(back["b"], t["b"])
    save_safetensors(str(tmp_path / "s.st"), {"x": torch.randn(2, 2).bfloat16()}, {"format": "pt"})
    st, md = load_safetensors(str(tmp_path / "s.st"))
    assert st["x"].dtype == torch.bfloat16 and md["format"] == "pt"

"""Hugging Face bridge (the reference's ``integrations/huggingface``: ``from_huggingface``, ``to_huggingface``,
``pipeline``, ``load_hf_dataset``; ``hf_integration.py``: ``load_hf_model`` / ``save_hf_model``).  Works on local
directories in the HF layout (config.json + *.safetensors); nothing is downloaded."""
from __future__ import annotations

import glob
import json
import os
from typing import Dict

import torch

from ..models import ModelConfig, build_model
from .formats import load_safetensors, save_safetensors
from .model_hub import map_hf_name

_HF_CFG = {"hidden_size": "hidden_size", "intermediate_size": "intermediate_size", "num_hidden_layers": "num_hidden_layers",
           "num_attention_heads": "num_attention_heads", "num_key_value_heads": "num_key_value_heads",
           "vocab_size": "vocab_size", "max_position_embeddings": "max_position_embeddings", "rms_norm_eps": "rms_norm_eps",
           "rope_theta": "rope_theta", "tie_word_embeddings": "tie_word_embeddings", "sliding_window": "sliding_window"}


def config_from_hf(hf_cfg: dict) -> ModelConfig:
    d = {ours: hf_cfg[theirs] for theirs, ours in _HF_CFG.items() if hf_cfg.get(theirs) is not None}
    d["architecture"] = "transformer"
    return ModelConfig.from_dict(d)


def _fuse(hf: Dict[str, torch.Tensor], cfg: ModelConfig) -> Dict[str, torch.Tensor]:
    """HF per-projection tensors -> this package's fused qkv / gate_up layout, via the reference-format names."""
    ref = {}
    for k, v in hf.items():
        name = map_hf_name(k)
        if name:
            ref[name] = v
    return ref


def from_huggingface(path: str, dtype=None, device=None):
    hf_cfg = json.load(open(os.path.join(path, "config.json")))
    cfg = config_from_hf(hf_cfg)
    model = build_model(cfg, dtype=dtype, device=device)
    tensors = {}
    for f in sorted(glob.glob(os.path.join(path, "*.safetensors"))):
        tensors.update(load_safetensors(f)[0])
    model.load_reference_state_dict(_fuse(tensors, cfg), strict=False)
    return model


load_hf_model = from_huggingface


def to_huggingface(model, path: str):
    """Writes config.json + model.safetensors with HF Llama tensor names."""
    os.makedirs(path, exist_ok=True)
    cfg = model.config
    hf_cfg = {theirs: getattr(cfg, ours) for theirs, ours in _HF_CFG.items() if hasattr(cfg, ours)}
    hf_cfg.update(architectures=["LlamaForCausalLM"], model_type="llama", torch_dtype="bfloat16")
    json.dump(hf_cfg, open(os.path.join(path, "config.json"), "w"), indent=1)
    out = {}
    for k, v in model.to_reference_state_dict().items():
        out[_to_hf_name(k)] = v.detach().cpu().contiguous()
    save_safetensors(os.path.join(path, "model.safetensors"), out, {"format": "pt"})
    return path


save_hf_model = to_huggingface


def _to_hf_name(ref: str) -> str:
    table = {"embedding": "model.embed_tokens.weight", "norm": "model.norm.weight", "lm_head": "lm_head.weight"}
    if ref in table:
        return table[ref]
    _, i, rest = ref.split(".", 2)
    sub = {"attn_norm.weight": "input_layernorm.weight", "mlp_norm.weight": "post_attention_layernorm.weight"}.get(
        rest, rest.replace("attn.", "self_attn."))
    return f"model.layers.{i}.{sub}"


class TextGenerationPipeline:
    def __init__(self, model, tokenizer):
        self.model, self.tok = model, tokenizer

    @torch.no_grad()
    def __call__(self, prompt: str, max_new_tokens=32, **kw):
        from ..serving.generation import generate
        dev = next(self.model.parameters()).device
        ids = torch.tensor([self.tok.encode(prompt)], device=dev)
        out = generate(self.model, ids, max_new_tokens, **kw)
        return [{"generated_text": self.tok.decode(out[0].tolist())}]


def pipeline(task: str, model, tokenizer=None):
    if task != "text-generation":
        raise ValueError("only 'text-generation' is supported")
    if tokenizer is None:
        from ..serving.server import ByteTokenizer
        tokenizer = ByteTokenizer(model.config.vocab_size)
    return TextGenerationPipeline(model, tokenizer)


def load_hf_dataset(path: str, text_field="text", split=None):
    """Local dataset files in the layouts ``datasets`` writes most often: .jsonl / .json / .txt / .parquet."""
    if path.endswith(".parquet"):
        import pyarrow.parquet as pq
        return pq.read_table(path).column(text_field).to_pylist()
    if path.endswith(".jsonl"):
        return [json.loads(line)[text_field] for line in open(path) if line.strip()]
    if path.endswith(".json"):
        d = json.load(open(path))
        d = d[split] if split and isinstance(d, dict) else d
        return [r[text_field] if isinstance(r, dict) else r for r in d]
    return [line.rstrip("\n") for line in open(path)]

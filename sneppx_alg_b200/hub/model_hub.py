"""Model zoo / hub API: ``from_pretrained`` (config + parameter estimate for a preset id, or a model with weights from
a local directory), ``ModelHub.from_pretrained / save_pretrained``, Hugging Face name mapping and conversion to
`.sneppx` in the reference's fixed tensor order (interface_bindings/model_zoo.py:1049-1268, 1380-1516), and a local
``Hub`` facade (load / search / list_models / download / upload; model_hub/hub.py:51-297)."""
from __future__ import annotations

import json
import os
import re
import shutil
from typing import Dict, List, Optional

import torch

from ..checkpoint.sneppx_format import load_tensors, save_tensors
from ..models import ModelConfig, build_model, config_from_name
from .formats import load_safetensors, save_safetensors

HF_WEIGHT_MAP = [
    (r"^model\.embed_tokens\.weight$", "embedding"),
    (r"^model\.norm\.weight$", "norm"),
    (r"^lm_head\.weight$", "lm_head"),
    (r"^model\.layers\.(\d+)\.input_layernorm\.weight$", r"layers.\1.attn_norm.weight"),
    (r"^model\.layers\.(\d+)\.post_attention_layernorm\.weight$", r"layers.\1.mlp_norm.weight"),
    (r"^model\.layers\.(\d+)\.self_attn\.([qkvo])_proj\.weight$", r"layers.\1.attn.\2_proj.weight"),
    (r"^model\.layers\.(\d+)\.mlp\.(gate|up|down)_proj\.weight$", r"layers.\1.mlp.\2_proj.weight"),
]


def map_hf_name(name: str) -> Optional[str]:
    for pat, rep in HF_WEIGHT_MAP:
        if re.match(pat, name):
            return re.sub(pat, rep, name)
    return None


def reference_tensor_order(num_layers: int) -> List[str]:
    names = ["embedding", "norm", "lm_head"]
    for i in range(num_layers):
        p = f"layers.{i}."
        names += [p + "attn_norm.weight", p + "attn.q_proj.weight", p + "attn.k_proj.weight", p + "attn.v_proj.weight",
                  p + "attn.o_proj.weight", p + "mlp_norm.weight", p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight",
                  p + "mlp.down_proj.weight"]
    return names


def convert_hf_to_sneppx(hf_state: Dict[str, torch.Tensor], out_path: str, config: ModelConfig, family: str = "llama"):
    """Rename HF tensors, order them as the reference does, write fp32 `.sneppx` with its metadata keys."""
    mapped = {}
    for k, v in hf_state.items():
        n = map_hf_name(k)
        if n is not None:
            mapped[n] = v
    if "lm_head" not in mapped and "embedding" in mapped:
        mapped["lm_head"] = mapped["embedding"]
    order = [n for n in reference_tensor_order(config.num_hidden_layers) if n in mapped]
    save_tensors(out_path, {n: mapped[n].float() for n in order},
                 {"family": family, "num_layers": config.num_hidden_layers, "num_converted": len(order),
                  "model_config": config.to_dict()})
    return order


def from_pretrained(name_or_path: str, dtype=None, device=None, **overrides):
    """Preset id -> dict {config, num_parameters, ...} like the reference; a directory with ``config.json`` and weights
    (`model.sneppx` or `model.safetensors`) -> a model instance with the weights loaded."""
    if os.path.isdir(name_or_path):
        return ModelHub.from_pretrained(name_or_path, dtype=dtype, device=device)
    cfg = config_from_name(name_or_path)
    for k, v in overrides.items():
        setattr(cfg, k, v)
    n = cfg.estimate_parameters()
    return {"name": cfg.name, "config": cfg, "num_parameters": n, "size_gb_bf16": n * 2 / 2 ** 30,
            "size_gb_train_adamw": n * 16 / 2 ** 30}


class ModelHub:
    @staticmethod
    def save_pretrained(model, directory: str, fmt: str = "sneppx"):
        os.makedirs(directory, exist_ok=True)
        model.config.to_json(os.path.join(directory, "config.json"))
        sd = model.to_reference_state_dict() if hasattr(model, "to_reference_state_dict") else model.state_dict()
        if fmt == "safetensors":
            save_safetensors(os.path.join(directory, "model.safetensors"), {k: v.contiguous() for k, v in sd.items()})
        else:
            save_tensors(os.path.join(directory, "model.sneppx"), sd, {"model_config": model.config.to_dict()})
        return directory

    @staticmethod
    def from_pretrained(directory: str, dtype=None, device=None):
        cfg = ModelConfig.from_json(os.path.join(directory, "config.json"))
        model = build_model(cfg, dtype=dtype, device=device)
        st = os.path.join(directory, "model.safetensors")
        sd = load_safetensors(st)[0] if os.path.exists(st) else load_tensors(os.path.join(directory, "model.sneppx"))[0]
        if any(k.startswith("model.layers.") for k in sd):     # raw Hugging Face names
            sd = {map_hf_name(k): v for k, v in sd.items() if map_hf_name(k)}
            sd.setdefault("lm_head", sd.get("embedding"))
        if hasattr(model, "load_reference_state_dict"):
            model.load_reference_state_dict(sd, strict=False)
        else:
            model.load_state_dict(sd, strict=False)
        return model


class Hub:
    """Local-directory model registry with the reference hub's verbs."""

    def __init__(self, root: str = "~/.sneppx/hub"):
        self.root = os.path.expanduser(root)
        os.makedirs(self.root, exist_ok=True)

    def _index(self):
        p = os.path.join(self.root, "index.json")
        return json.load(open(p)) if os.path.exists(p) else {}

    def _write_index(self, idx):
        with open(os.path.join(self.root, "index.json"), "w") as f:
            json.dump(idx, f, indent=2)

    def upload(self, model_dir: str, model_id: str, version: str = "1.0.0", tags=(), metrics: dict = None):
        dst = os.path.join(self.root, model_id.replace("/", "__"), version)
        if os.path.exists(dst):
            shutil.rmtree(dst)
        shutil.copytree(model_dir, dst)
        idx = self._index()
        idx.setdefault(model_id, {})[version] = {"path": dst, "tags": list(tags), "metrics": metrics or {}}
        self._write_index(idx)
        return dst

    def download(self, model_id: str, version: Optional[str] = None) -> str:
        vs = self._index()[model_id]
        return vs[version or sorted(vs)[-1]]["path"]

    def load(self, model_id: str, version: Optional[str] = None, **kw):
        return ModelHub.from_pretrained(self.download(model_id, version), **kw)

    def list_models(self):
        return {m: sorted(v) for m, v in self._index().items()}

    def search(self, query: str = "", tag: Optional[str] = None):
        return [m for m, vs in self._index().items()
                if query.lower() in m.lower() and (tag is None or any(tag in v["tags"] for v in vs.values()))]

    def leaderboard(self, metric: str, higher_is_better=True):
        rows = [(m, v, info["metrics"][metric]) for m, vs in self._index().items() for v, info in vs.items()
                if metric in info["metrics"]]
        return sorted(rows, key=lambda r: r[2], reverse=higher_is_better)

"""Model configuration and the preset zoo.

``ModelConfig`` carries the field names of the reference's unified schema
(interface_bindings/model_zoo.py:16-99, include/neural_core/kernel/model_config.h) so that its JSON
files load unchanged; the presets reproduce the reference registry (model_zoo.py:824-948,
kernel/model_zoo/model_zoo.c:197) and add the HSS / SER shapes used by the benchmarks.
"""
from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field
from typing import Any, Dict, Optional


@dataclass
class ModelConfig:
    # identity
    name: str = ""
    version: str = "0.1.0"
    description: str = ""
    author: str = ""
    license: str = ""
    repository: str = ""
    homepage: str = ""
    architecture: str = "transformer"   # transformer | mamba2 | hss_ser | deepseek_moe | bert | gpt | t5 | vit
    model_type: str = "causal-lm"
    framework: str = "sneppx"
    # shape
    num_parameters: int = 0
    num_layers: int = 0
    num_hidden_layers: int = 0
    hidden_size: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0
    vocab_size: int = 0
    max_seq_len: int = 0
    max_position_embeddings: int = 0
    # norms / activations
    layer_norm_eps: float = 1e-5
    rms_norm_eps: float = 1e-6
    use_rms_norm: bool = True
    hidden_act: str = "silu"
    ffn_act: str = "silu"
    gated_ffn: bool = True
    # attention
    attention_type: str = "causal"
    attention_dropout: float = 0.0
    hidden_dropout: float = 0.0
    use_flash_attention: bool = True
    sliding_window: int = 0
    differential_attention: bool = False
    # positions
    pos_encoding: str = "rope"
    rope_theta: float = 10000.0
    rope_scaling: Any = 0
    rope_scale_factor: float = 1.0
    # init
    initializer_range: float = 0.02
    tie_word_embeddings: bool = False
    # quantisation
    quantize: bool = False
    quant_bits: int = 0
    quant_group_size: int = 128
    # distributed
    tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    expert_parallel_size: int = 1
    sequence_parallel: bool = False
    # training defaults
    learning_rate: float = 2e-4
    weight_decay: float = 0.01
    max_grad_norm: float = 1.0
    warmup_steps: int = 0
    max_steps: int = 0
    gradient_accumulation_steps: int = 1
    mixed_precision: bool = True
    # MoE (SER)
    num_experts: int = 0
    num_experts_per_token: int = 0
    num_shared_experts: int = 0
    moe_intermediate_size: int = 0
    first_dense_layers: int = 0
    router_aux_loss_coef: float = 0.0
    router_z_loss_coef: float = 0.0
    expert_capacity_factor: float = 0.0   # 0: dropless
    expert_fp8: bool = False              # forward expert GEMMs in block-scaled e4m3 (1x128 / 128x128 scales)
    fp8_experts: bool = False
    # MLA (DeepSeek-V2)
    kv_lora_rank: int = 0
    q_lora_rank: int = 0
    # SSM (HSS / Mamba-2)
    ssm_state_size: int = 0
    ssm_expand: int = 2
    ssm_head_dim: int = 64
    ssm_ngroups: int = 1
    ssm_conv_kernel: int = 4
    ssm_chunk_size: int = 256
    custom: Dict[str, Any] = field(default_factory=dict)

    def __post_init__(self):
        if not self.num_hidden_layers and self.num_layers:
            self.num_hidden_layers = self.num_layers
        if not self.num_layers and self.num_hidden_layers:
            self.num_layers = self.num_hidden_layers
        if not self.max_seq_len and self.max_position_embeddings:
            self.max_seq_len = self.max_position_embeddings
        if not self.max_position_embeddings and self.max_seq_len:
            self.max_position_embeddings = self.max_seq_len
        if not self.num_key_value_heads:
            self.num_key_value_heads = self.num_attention_heads
        if not self.head_dim and self.num_attention_heads:
            self.head_dim = self.hidden_size // self.num_attention_heads

    # ---- (de)serialisation
    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)

    def to_json(self, path: Optional[str] = None, indent: int = 2) -> str:
        s = json.dumps(self.to_dict(), indent=indent)
        if path:
            with open(path, "w") as f:
                f.write(s)
        return s

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ModelConfig":
        names = {f.name for f in dataclasses.fields(cls)}
        known = {k: v for k, v in d.items() if k in names}
        extra = {k: v for k, v in d.items() if k not in names}
        cfg = cls(**known)
        cfg.custom.update(extra)
        return cfg

    @classmethod
    def from_json(cls, path_or_text: str) -> "ModelConfig":
        text = path_or_text
        if not path_or_text.lstrip().startswith("{"):
            with open(path_or_text) as f:
                text = f.read()
        return cls.from_dict(json.loads(text))

    def validate(self):
        errs = []
        if self.architecture in ("transformer", "deepseek_moe"):
            if self.hidden_size <= 0 or self.num_attention_heads <= 0:
                errs.append("hidden_size and num_attention_heads must be positive")
            elif self.num_attention_heads % max(self.num_key_value_heads, 1):
                errs.append("num_attention_heads must be a multiple of num_key_value_heads")
        if self.vocab_size <= 0:
            errs.append("vocab_size must be positive")
        if self.num_experts and not (0 < self.num_experts_per_token <= self.num_experts):
            errs.append("num_experts_per_token must be in (0, num_experts]")
        return errs

    def estimate_parameters(self) -> int:
        d, L, V = self.hidden_size, self.num_hidden_layers, self.vocab_size
        hd = self.head_dim or 0
        attn = d * (self.num_attention_heads + 2 * self.num_key_value_heads) * hd + self.num_attention_heads * hd * d
        ffn = (3 if self.gated_ffn else 2) * d * self.intermediate_size
        if self.architecture == "mamba2":
            di = self.ssm_expand * d
            nh = di // self.ssm_head_dim
            per = d * (2 * di + 2 * self.ssm_ngroups * self.ssm_state_size + nh) + di * d + 2 * d
            return L * per + V * d
        if self.num_experts:
            moe = (3 * d * self.moe_intermediate_size) * (self.num_experts + self.num_shared_experts) + d * self.num_experts
            dense = self.first_dense_layers
            total = dense * (attn + ffn) + (L - dense) * (attn + moe)
        else:
            total = L * (attn + ffn)
        emb = V * d * (1 if self.tie_word_embeddings else 2)
        return total + emb + (2 * L + 1) * d


class LlamaConfig(ModelConfig):
    pass


class MistralConfig(ModelConfig):
    pass


class Qwen2Config(ModelConfig):
    pass


class DeepSeekV2Config(ModelConfig):
    pass


def _tf(**kw):
    return dict(architecture="transformer", **kw)


_MODEL_REGISTRY: Dict[str, Dict[str, dict]] = {
    "llama2": {
        "7B": _tf(hidden_size=4096, intermediate_size=11008, num_hidden_layers=32, num_attention_heads=32,
                  num_key_value_heads=32, vocab_size=32000, max_position_embeddings=4096, rope_theta=1e4, rms_norm_eps=1e-5),
        "13B": _tf(hidden_size=5120, intermediate_size=13824, num_hidden_layers=40, num_attention_heads=40,
                   num_key_value_heads=40, vocab_size=32000, max_position_embeddings=4096, rope_theta=1e4, rms_norm_eps=1e-5),
        "70B": _tf(hidden_size=8192, intermediate_size=28672, num_hidden_layers=80, num_attention_heads=64,
                   num_key_value_heads=8, vocab_size=32000, max_position_embeddings=4096, rope_theta=1e4, rms_norm_eps=1e-5),
    },
    "llama3": {
        "tiny": _tf(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                    num_key_value_heads=1, head_dim=64, vocab_size=512, max_position_embeddings=512, rope_theta=1e4,
                    rms_norm_eps=1e-5),
        "8B": _tf(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                  num_key_value_heads=8, vocab_size=128256, max_position_embeddings=8192, rope_theta=5e5, rms_norm_eps=1e-5),
        "70B": _tf(hidden_size=8192, intermediate_size=28672, num_hidden_layers=80, num_attention_heads=64,
                   num_key_value_heads=8, vocab_size=128256, max_position_embeddings=8192, rope_theta=5e5, rms_norm_eps=1e-5),
    },
    "mistral": {
        "7B": _tf(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                  num_key_value_heads=8, vocab_size=32000, max_position_embeddings=32768, sliding_window=4096,
                  rope_theta=1e4, rms_norm_eps=1e-5),
    },
    "qwen2": {
        "7B": _tf(hidden_size=3584, intermediate_size=18944, num_hidden_layers=28, num_attention_heads=28,
                  num_key_value_heads=4, vocab_size=152064, max_position_embeddings=32768, rope_theta=1e6),
        "72B": _tf(hidden_size=8192, intermediate_size=29568, num_hidden_layers=80, num_attention_heads=64,
                   num_key_value_heads=8, vocab_size=152064, max_position_embeddings=32768, rope_theta=1e6),
    },
    "deepseek_v2": {
        "lite": dict(architecture="deepseek_moe", hidden_size=2048, intermediate_size=10944, num_hidden_layers=27,
                     num_attention_heads=16, num_key_value_heads=16, head_dim=128, vocab_size=102400,
                     max_position_embeddings=4096, kv_lora_rank=512, q_lora_rank=1536, rope_theta=1e4,
                     rms_norm_eps=1e-6, num_experts=64, num_experts_per_token=6, num_shared_experts=2,
                     moe_intermediate_size=1408, first_dense_layers=1, router_aux_loss_coef=0.001),
        "full": dict(architecture="deepseek_moe", hidden_size=5120, intermediate_size=12288, num_hidden_layers=60,
                     num_attention_heads=64, num_key_value_heads=64, head_dim=128, vocab_size=102400,
                     max_position_embeddings=4096, kv_lora_rank=512, q_lora_rank=1536, rope_theta=1e4,
                     rms_norm_eps=1e-6, num_experts=160, num_experts_per_token=6, num_shared_experts=2,
                     moe_intermediate_size=1536, first_dense_layers=1, router_aux_loss_coef=0.001),
    },
    "mamba2": {
        "2.7B": dict(architecture="mamba2", hidden_size=2560, num_hidden_layers=64, vocab_size=50280,
                     ssm_state_size=128, ssm_expand=2, ssm_head_dim=64, ssm_ngroups=8, ssm_conv_kernel=4,
                     ssm_chunk_size=256, max_position_embeddings=8192, rms_norm_eps=1e-5, tie_word_embeddings=True),
        "130M": dict(architecture="mamba2", hidden_size=768, num_hidden_layers=24, vocab_size=50280,
                     ssm_state_size=128, ssm_expand=2, ssm_head_dim=64, ssm_ngroups=1, ssm_conv_kernel=4,
                     ssm_chunk_size=256, max_position_embeddings=8192, rms_norm_eps=1e-5, tie_word_embeddings=True),
    },
    "hss_ser": {
        "tiny": dict(architecture="hss_ser", hidden_size=256, num_hidden_layers=4, vocab_size=32000,
                     ssm_state_size=64, ssm_expand=2, ssm_head_dim=64, ssm_ngroups=1, ssm_conv_kernel=4,
                     ssm_chunk_size=64, num_experts=8, num_experts_per_token=2, moe_intermediate_size=512,
                     expert_capacity_factor=1.25, router_aux_loss_coef=0.01, max_position_embeddings=512,
                     rms_norm_eps=1e-5, tie_word_embeddings=True),
    },
}

_ALIASES = {"llama": "llama2", "llama-2": "llama2", "llama-3": "llama3", "deepseek": "deepseek_v2",
            "deepseek-v2": "deepseek_v2", "mamba-2": "mamba2", "hss": "hss_ser"}


def list_models():
    return {fam: sorted(sizes) for fam, sizes in _MODEL_REGISTRY.items()}


def get_model_config(family: str, size: str) -> dict:
    """Preset as a plain dict (the reference's ``get_model_config`` contract, model_zoo.py:951)."""
    fam = family.lower().replace(" ", "")
    fam = _ALIASES.get(fam, fam).replace("-", "_")
    if fam not in _MODEL_REGISTRY:
        raise ValueError(f"Unknown model family '{family}'. Available: {sorted(_MODEL_REGISTRY)}")
    sizes = _MODEL_REGISTRY[fam]
    key = next((k for k in sizes if k.lower() == str(size).lower()), None)
    if key is None:
        raise ValueError(f"Unknown size '{size}' for '{fam}'. Available: {sorted(sizes)}")
    return dict(sizes[key])


def config_from_name(name: str) -> ModelConfig:
    """'llama3-8b', 'meta-llama/Llama-3-8B', 'mistral-7b', 'deepseek-v2-lite', 'mamba2-2.7b', 'hss-ser-tiny' ..."""
    n = name.lower().split("/")[-1].replace("_", "-")
    table = [("llama-3", "llama3"), ("llama3", "llama3"), ("llama-2", "llama2"), ("llama2", "llama2"),
             ("llama", "llama2"), ("mistral", "mistral"), ("qwen2", "qwen2"), ("deepseek", "deepseek_v2"),
             ("mamba", "mamba2"), ("hss", "hss_ser")]
    for pat, fam in table:
        if pat in n:
            for size in _MODEL_REGISTRY[fam]:
                if size.lower() in n:
                    cfg = ModelConfig.from_dict(get_model_config(fam, size))
                    cfg.name = f"{fam}-{size}"
                    return cfg
            size = next(iter(_MODEL_REGISTRY[fam]))
            cfg = ModelConfig.from_dict(get_model_config(fam, size))
            cfg.name = f"{fam}-{size}"
            return cfg
    raise ValueError(f"cannot infer a preset from '{name}'")


def extend_context(cfg: ModelConfig, new_len: int, method: str = "ntk") -> ModelConfig:
    """RoPE context extension (linear / NTK / YaRN-style), the reference's ``extend_context``
    (model_zoo.py:998-1033, kernel/model_zoo/model_zoo.c:496)."""
    out = dataclasses.replace(cfg)
    base = cfg.max_position_embeddings or cfg.max_seq_len
    if new_len <= base:
        return out
    scale = new_len / base
    out.max_position_embeddings = out.max_seq_len = new_len
    out.rope_scaling = method
    out.rope_scale_factor = scale
    return out

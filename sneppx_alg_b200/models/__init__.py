"""Model families and the preset zoo."""
from .config import (ModelConfig, LlamaConfig, MistralConfig, Qwen2Config, DeepSeekV2Config, get_model_config,  # noqa: F401
                     config_from_name, extend_context, list_models)
from .llama import LlamaForCausalLM, MistralForCausalLM, Qwen2ForCausalLM, create_model  # noqa: F401


def build_model(cfg, dtype=None, device=None):
    """Instantiate the model class that ``cfg.architecture`` names."""
    arch = cfg.architecture
    if arch == "transformer":
        return LlamaForCausalLM(cfg, dtype=dtype, device=device)
    if arch == "mamba2":
        from .mamba2 import Mamba2ForCausalLM
        return Mamba2ForCausalLM(cfg, dtype=dtype, device=device)
    if arch == "hss_ser":
        from .hss_ser import HSSSERForCausalLM
        return HSSSERForCausalLM(cfg, dtype=dtype, device=device)
    if arch == "deepseek_moe":
        from .deepseek import DeepSeekV2ForCausalLM
        return DeepSeekV2ForCausalLM(cfg, dtype=dtype, device=device)
    raise ValueError(f"unknown architecture '{arch}'")

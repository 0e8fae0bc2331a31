"""Model hub: presets, from_pretrained, weight formats, local registry."""
from .formats import (load_hub_container, load_npz, load_safetensors, save_hub_container, save_npz,  # noqa: F401
                      save_safetensors)
from .model_hub import (HF_WEIGHT_MAP, Hub, ModelHub, convert_hf_to_sneppx, from_pretrained, map_hf_name,  # noqa: F401
                        reference_tensor_order)

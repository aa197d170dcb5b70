from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from .qwen3 import ConfigError, Qwen3Config
from .lederax import LederaxConfig
from .vunepel import VunepelConfig
from .bisodra import BisodraConfig
from .regupel import RegupelConfig
from .registry import (
    config_from_dict,
    load_config,
    load_config_dict,
    load_preset,
    preset_names,
    register_architecture,
    registered_architectures,
)

register_architecture("Qwen3ForCausalLM", Qwen3Config, model_type="qwen3")
register_architecture("Lederax", LederaxConfig)
register_architecture("Vunepel", VunepelConfig)
register_architecture("Bisodra", BisodraConfig)
register_architecture("Regupel", RegupelConfig)

__all__ = [
    "BisodraConfig", "ConfigError", "LayerCall", "LayerSpec", "LederaxConfig", "ModelSpec", "PartSpec", "Qwen3Config", "RegupelConfig", "VunepelConfig",
    "config_from_dict", "load_config", "load_config_dict", "load_preset", "preset_names",
    "register_architecture", "registered_architectures",
]

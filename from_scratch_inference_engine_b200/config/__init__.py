from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from .qwen2 import ConfigError, Qwen2Config
from .registry import (architecture_name, config_from_dict, load_config, register_architecture,
                       registered_architectures, unregister_architecture)

__all__ = [
    "LayerCall", "LayerSpec", "ModelSpec", "PartSpec", "ConfigError", "Qwen2Config",
    "architecture_name", "config_from_dict", "load_config", "register_architecture",
    "registered_architectures", "unregister_architecture",
]

from .spec import CallSpec, ConfigError, LayerSpec, ModelSpec, PartSpec, SubLayerSpec
from .registry import config_from_dict, known_architectures, load_config, register_architecture
from .qwen2 import Qwen2Config

__all__ = ["CallSpec", "ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "SubLayerSpec", "Qwen2Config",
           "config_from_dict", "known_architectures", "load_config", "register_architecture"]

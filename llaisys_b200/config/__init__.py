from .spec import CallSpec, ConfigError, LayerSpec, ModelSpec, PartSpec, SubLayerSpec
from .registry import config_from_dict, known_architectures, load_config, register_architecture
from .qwen2 import Qwen2Config
from .vumezen import VumezenConfig

__all__ = ["CallSpec", "ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "SubLayerSpec", "Qwen2Config", "VumezenConfig",
           "config_from_dict", "known_architectures", "load_config", "register_architecture"]

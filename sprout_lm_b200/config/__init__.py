from .specs import ConfigError, LayerCall, LayerSpec, ModelSpec, PartSpec
from .registry import (architecture_name, load_config, parse_config, register_architecture,
                       registered_architectures)
from .qwen2 import Qwen2Config
from .tulipel import TulipelConfig
from .letanex import LetanexConfig

register_architecture(Qwen2Config.architecture, Qwen2Config, model_types=(Qwen2Config.model_type,))
register_architecture(TulipelConfig.architecture, TulipelConfig)
register_architecture(LetanexConfig.architecture, LetanexConfig)

__all__ = ["ConfigError", "LayerCall", "LayerSpec", "ModelSpec", "PartSpec", "Qwen2Config", "TulipelConfig", "LetanexConfig",
           "architecture_name", "load_config", "parse_config", "register_architecture",
           "registered_architectures"]

from .base import (ConfigError, LayerSpec, ModelConfig, ModelPlan, PartSpec, ScheduleEntry,
                   UnsupportedError)
from .registry import (config_from_dict, config_from_gguf, known_architectures, load_config, register_architecture,
                       unregister_architecture)
from .qwen2 import Qwen2Config

__all__ = ["ConfigError", "UnsupportedError", "ModelConfig", "ModelPlan", "PartSpec", "LayerSpec",
           "ScheduleEntry", "Qwen2Config", "config_from_dict", "config_from_gguf", "load_config",
           "register_architecture", "unregister_architecture", "known_architectures"]

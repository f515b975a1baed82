from .base import (ConfigError, ModelConfig, build_model_spec, known_architectures, load_config,
                   lookup_architecture, parse_config, register_architecture)
from .llama import LlamaConfig
from .nutizen import NutizenConfig
from .ronurax import RonuraxConfig
from .sozarax import SozaraxConfig

__all__ = ["ConfigError", "ModelConfig", "LlamaConfig", "NutizenConfig", "RonuraxConfig", "SozaraxConfig", "build_model_spec", "known_architectures",
           "load_config", "lookup_architecture", "parse_config", "register_architecture"]

from .base import ConfigError
from .llama import LlamaConfig, RopeScaling
from .registry import (Architecture, architecture_for, load_config, register_architecture,
                       registered_architectures)

__all__ = ["ConfigError", "LlamaConfig", "RopeScaling", "Architecture", "architecture_for", "load_config",
           "register_architecture", "registered_architectures"]

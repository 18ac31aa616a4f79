from .base import ConfigError, read_json
from .llama import LlamaConfig, RopeScaling
from .registry import (Architecture, load_config, register_architecture,
                       registered_architectures, resolve_architecture)

__all__ = ["ConfigError", "read_json", "LlamaConfig", "RopeScaling", "Architecture",
           "load_config", "register_architecture", "registered_architectures",
           "resolve_architecture"]

from .model_config import ConfigError, Qwen2Config, architecture_name, read_config_json
from .registry import (Architecture, register_architecture, unregister_architecture,
                       registered_architectures, resolve_architecture, load_config)
from .options import EngineOptions

__all__ = [
    "ConfigError", "Qwen2Config", "architecture_name", "read_config_json", "Architecture",
    "register_architecture", "unregister_architecture", "registered_architectures",
    "resolve_architecture", "load_config", "EngineOptions",
]

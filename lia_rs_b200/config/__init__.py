from .model_config import ConfigError, LlamaConfig, read_config_json
from .registry import Architecture, known_architectures, register_architecture, resolve_architecture

__all__ = ["ConfigError", "LlamaConfig", "read_config_json", "Architecture",
           "known_architectures", "register_architecture", "resolve_architecture"]

"""Typed configurations and the architecture registry."""
from .fields import ConfigError, KeyReader, read_config_json
from .llama import LlamaConfig
from .registry import (Architecture, register_architecture, registered_names,
                       resolve_architecture, unregister_architecture)

__all__ = ["ConfigError", "KeyReader", "read_config_json", "LlamaConfig", "Architecture",
           "register_architecture", "registered_names", "resolve_architecture",
           "unregister_architecture"]

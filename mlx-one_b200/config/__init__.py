from .base import ConfigError
from .lfm2 import Lfm2Config
from .registry import (Architecture, architecture_names, get_architecture, read_config,
                       register_architecture, unregister_architecture)

__all__ = ["ConfigError", "Lfm2Config", "Architecture", "architecture_names",
           "get_architecture", "read_config", "register_architecture",
           "unregister_architecture"]

from .base import ConfigError, ConfigReader, read_config_json, architecture_name
from .hunyuan_dense import HunyuanDenseConfig
from .registry import (Architecture, register_architecture, get_architecture,
                       known_architectures, load_config)

__all__ = ["ConfigError", "ConfigReader", "read_config_json", "architecture_name", "HunyuanDenseConfig",
           "Architecture", "register_architecture", "get_architecture", "known_architectures", "load_config"]

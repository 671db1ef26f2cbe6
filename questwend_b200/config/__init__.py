from .base import ConfigError, ConfigReader, ModelConfig, read_config_json
from .registry import (Architecture, register_architecture, get_architecture, architectures,
                       architecture_name, config_from_dict, load_config)

__all__ = ["ConfigError", "ConfigReader", "ModelConfig", "read_config_json", "Architecture",
           "register_architecture", "get_architecture", "architectures", "architecture_name",
           "config_from_dict", "load_config"]

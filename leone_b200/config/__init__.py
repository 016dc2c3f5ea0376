from .base import (ConfigError, InvalidValue, MissingKey, ModelConfig, UnsupportedArchitecture,
                   UnsupportedField, WrongType, read_config_json)
from .qwen3 import Qwen3Config

__all__ = ["ConfigError", "InvalidValue", "MissingKey", "ModelConfig", "UnsupportedArchitecture",
           "UnsupportedField", "WrongType", "read_config_json", "Qwen3Config"]
